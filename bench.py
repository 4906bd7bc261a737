"""Benchmark of the GatedDeltaNet / GQA-decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Headline line (one JSON object on stdout, rank 0):
  metric   decode steps/s at B=64 -- one step = one token for each of 64 sequences through the model's 18 GatedDeltaNet layers
           (benchmark configuration 2: conv1d k=4 over the mixed qkv row, q/k l2norm, gates, gated delta rule on the fp32
           [16,128,128] state, in-place slot pools).  With N GPUs the batch is sharded by sequence: every GPU owns its own 64
           sequences (weak scaling, no collective on the data path) and `value` is the sum over GPUs.
  value    kernel-only throughput, state pools and inputs resident in HBM, the 18 launches of a step replayed from a CUDA graph;
           the K-step timed region is repeated and the median region is reported.
  e2e      the same step through the Python operator API with the step's inputs (proj rows) in pinned host memory and the outputs
           read back to the host inside the timed region, one packed copy per direction, step n+1 enqueued before step n is read.
  roofline HBM roofline of the decode kernel: algorithmic bytes per launch / average launch time, against the measured copy bandwidth.
  extra    further workloads of the hot path (chunked prefill at T=2048 x 18 layers and T=8192, the ragged batch of configuration 4,
           speculative verify + paged GQA attention of configuration 5, decode at B=1/16), each with its own roofline fraction and
           the device status word it left behind.  At N=1 they run in a child process, so a failure there cannot lose the headline.
`--impl reference` times the CPU restatement of the reference's arithmetic (OpenMP C port, all host threads) on the same step.
"""
from __future__ import annotations

import argparse
import copy
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
import traceback
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

HV, DK, DV, CD, PW = 16, 128, 128, 6144, 8224
N_LAYERS = 18
B_DECODE = 64
STATE_BYTES = HV * DV * DK * 4
# algorithmic bytes of one decode step of one (sequence, layer): state read + state written + mixed-qkv row + conv window read
# + conv window written + y  (M = 1)
DECODE_BYTES_PER_SEQ_LAYER = 2 * STATE_BYTES + CD * 2 + 3 * CD * 2 + 3 * CD * 2 + HV * DV * 2
# dram__bytes_read.sum + dram__bytes_write.sum of one decode launch at B=64 from an ncu capture of this kernel (70.35 MB read +
# 11.57 MB written; the rest of the 67 MB of state written by a launch is still in L2 when the kernel ends and is written back
# during the following launches)
DECODE_TRAFFIC_NCU = 81920000
PREFILL_FLOP_PER_TOKEN_LAYER = HV * (8 * 64 * 128 + 6 * 128 * 128)        # chunk 64: 2,621,440
PREFILL_BYTES_PER_TOKEN_LAYER = 4 * HV * 128 * 2 + 2 * HV * 4                # q,k,v,y bf16 + log-decay, beta fp32 = 16,512
# values of the device status word (a kernel that meets one of these skips the row or leaves; nothing faults)
STATUS_NAMES = {0: "ok", 1: "index out of range (row skipped)", 2: "decode/attention wait gave up", 3: "prefill wait gave up",
                4: "shared memory misaligned"}
REGION_REPEATS = 5


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def read_status(_lib):
    code = _lib.device_status()
    return dict(code=code, meaning=STATUS_NAMES.get(code, "unknown"))


# ----------------------------------------------------------------------------------------------------------------------
# clocks sampling (nvidia-smi in the background during the timed region)
# ----------------------------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.split(", ") for r in Path(self.file.name).read_text().strip().splitlines() if r.strip()]
        os.unlink(self.file.name)
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2])); power.append(float(r[3]))
            except ValueError:
                continue
            for n, v in zip(names, r[5:9]):
                if v.strip().lower() == "active":
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples taken while the GPU was busy (power well above idle) describe the clock under load
        busy = [s for s, p in zip(sm, power) if p >= 0.6 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "power_w_max": max(power) if power else None}


# ----------------------------------------------------------------------------------------------------------------------
# timing
# ----------------------------------------------------------------------------------------------------------------------
def time_region(torch, fn, iters, dist=None, repeats=1, finish=None):
    """Run fn() `iters` times between CUDA events on the current stream, bracketed by barrier + synchronize; the region is repeated
    `repeats` times and the median is returned in ms (every region is the max over ranks).  `finish`, if given, is called after
    the last fn() of a region and before the closing event (it makes the current stream wait for work on side streams)."""
    out = []
    for _ in range(repeats):
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        if finish is not None:
            finish()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = float(t.item())
        out.append(ms)
    return statistics.median(out)


def graphed(torch, step, warm=3):
    """Run `step` a few times, capture it into a CUDA graph (as the reference compiles its step) and return the replay callable."""
    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    for _ in range(warm):
        g.replay()
    return g.replay


def rn_factory(torch, dev, seed):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return g, (lambda *s: torch.randn(s, generator=g, device=dev, dtype=torch.float32))


# ----------------------------------------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------------------------------------
def make_decode_layers(torch, dev, B, n_layers, seed, n_proj_sets=1):
    """Per-layer slot pools and inputs of benchmark configuration 2 (state ~ N(0, 0.02), everything else ~ N(0, 1)).  The proj rows
    and the outputs of all layers live in packed buffers ([sets, layers, B, .]) so that a step's inputs / outputs move in one copy."""
    g, _ = rn_factory(torch, dev, seed)
    proj_all = torch.randn((n_proj_sets, n_layers, B, PW), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    y_all = torch.zeros((n_proj_sets, n_layers, B, HV * DV), device=dev, dtype=torch.bfloat16)
    layers = []
    for _ in range(n_layers):
        layers.append(dict(
            conv_pool=torch.randn(((B + 1) * 2, 3, CD), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16),
            conv_w=(torch.randn((CD * 4,), generator=g, device=dev, dtype=torch.float32) * 0.5).to(torch.bfloat16),
            A_log=torch.rand((HV,), generator=g, device=dev, dtype=torch.float32) * math.log(16.0),
            dt_bias=(torch.randn((HV,), generator=g, device=dev, dtype=torch.float32) * 0.1).to(torch.bfloat16).float(),
            ssm_pool=torch.randn((B + 1, HV, DV, DK), generator=g, device=dev, dtype=torch.float32) * 0.02))
    return layers, proj_all, y_all


def bench_decode(torch, dev, args, dist, peaks, B=B_DECODE, n_layers=N_LAYERS, with_e2e=True):
    from qwen_tailor_b200.batch import deltanet_b
    sets = 2 if with_e2e else 1
    layers, proj_all, y_all = make_decode_layers(torch, dev, B, n_layers, seed=1 + (dist.get_rank() if dist else 0), n_proj_sets=sets)
    slots = torch.arange(B, dtype=torch.int32, device=dev)
    pos = torch.zeros(B, dtype=torch.int32, device=dev)

    def make_step(s):
        def step():
            for i, L in enumerate(layers):
                deltanet_b(proj_all[s, i], L["conv_pool"], L["conv_w"], L["A_log"], L["dt_bias"], L["ssm_pool"], slots, pos, out=y_all[s, i])
            pos.add_(1)                                   # flips the conv double buffer like a real decode loop
        return step

    graphs = []
    for s in range(sets):
        step = make_step(s)
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        graphs.append(g)
    for _ in range(max(args.warmup, 3)):
        graphs[0].replay()
    ms = time_region(torch, graphs[0].replay, args.steps, dist, repeats=REGION_REPEATS)
    ms_per_step = ms / args.steps
    launch_us = ms_per_step * 1e3 / n_layers
    gbs = B * DECODE_BYTES_PER_SEQ_LAYER / (launch_us * 1e-6) / 1e9
    out = dict(ms_per_step=ms_per_step, launch_us=launch_us, achieved_gbs=gbs, frac=gbs / peaks["hbm_gbs"], launches=args.steps * n_layers,
               state_gb=n_layers * (B + 1) * STATE_BYTES / 1e9)
    if with_e2e:
        # The caller's view of a step: proj rows of all layers start in pinned host memory, y of all layers ends there.  One packed
        # copy per direction; two input / output sets so that step n+1's upload and step n's download overlap step n's kernels,
        # as the reference's server enqueues step n+1 before it reads step n (qwen35/serve.py:479-503).
        host_in = [torch.randn((n_layers, B, PW), dtype=torch.float32).to(torch.bfloat16).pin_memory() for _ in range(2)]
        host_out = [torch.empty((n_layers, B, HV * DV), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        s_comp = torch.cuda.current_stream()
        s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()
        up_done = [torch.cuda.Event() for _ in range(2)]
        comp_done = [torch.cuda.Event() for _ in range(2)]
        down_done = [torch.cuda.Event() for _ in range(2)]
        n_issued = [0]

        def e2e_step():
            n = n_issued[0]
            s = n & 1
            s_up.wait_event(comp_done[s])                 # the kernels of step n-2 have finished reading this input set
            with torch.cuda.stream(s_up):
                proj_all[s].copy_(host_in[s], non_blocking=True)
                up_done[s].record(s_up)
            s_comp.wait_event(up_done[s])
            s_comp.wait_event(down_done[s])               # step n-2's outputs of this set have left the device
            graphs[s].replay()
            comp_done[s].record(s_comp)
            s_down.wait_event(comp_done[s])
            with torch.cuda.stream(s_down):
                host_out[s].copy_(y_all[s], non_blocking=True)
                down_done[s].record(s_down)
            if n >= 1:
                down_done[s ^ 1].synchronize()            # the caller reads step n-1's result while step n runs
            n_issued[0] = n + 1

        def finish():
            last = (n_issued[0] - 1) & 1
            down_done[last].synchronize()
            s_comp.wait_event(down_done[last])

        for _ in range(4):
            e2e_step()
        finish()
        ms_e = time_region(torch, e2e_step, args.steps, dist, repeats=REGION_REPEATS, finish=finish)
        out["e2e_ms_per_step"] = ms_e / args.steps
        out["h2d"] = n_layers * B * PW * 2
        out["d2h"] = n_layers * B * HV * DV * 2
    return out


def bench_attention(torch, dev, args, peaks, n_layers=6):
    """Configuration 5, attention part: B=16, M=4 rows per sequence, 6 layers, paged cache, ctx ~ U[1024, 8192]."""
    import numpy as np
    from qwen_tailor_b200 import synth
    from qwen_tailor_b200.batch import attn_paged
    ctx, _ = synth.config5_shapes()
    B, M, page = len(ctx), 4, 64
    need = (ctx.astype(np.int64) + M + page - 1) // page
    max_pages, n_pages = int(need.max()), int(need.sum()) + 1
    table = np.zeros((B, max_pages), np.int32)
    o = 1
    for i in range(B):
        table[i, :need[i]] = np.arange(o, o + need[i])
        o += need[i]
    g, _ = rn_factory(torch, dev, 11)
    rn = lambda *s: torch.randn(s, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    layers = [dict(K=rn(n_pages, 2, page, 256), V=rn(n_pages, 2, page, 256), q=rn(B * M, 8, 256), k=rn(B * M, 2, 256), v=rn(B * M, 2, 256))
              for _ in range(n_layers)]
    bt = torch.from_numpy(table).to(dev)
    cl = torch.from_numpy(ctx).to(dev)
    mc = int(ctx.max())

    def step():
        for L in layers:
            attn_paged(L["q"], L["k"], L["v"], L["K"], L["V"], bt, cl, M=M, max_ctx=mc)

    ms = time_region(torch, graphed(torch, step), args.steps, repeats=3) / args.steps
    byts = n_layers * float(ctx.sum()) * 2048
    gbs = byts / (ms * 1e-3) / 1e9
    return dict(workload=f"GQA decode attention, config 5: B=16, M=4, {n_layers} layers, paged bf16 KV, ctx~U[1024,8192]", ms_per_step=ms,
                kv_gb=byts / 1e9, roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"]))


def bench_attention_large(torch, dev, args, peaks, B=64, ctx=8192, n_layers=2):
    """The same kernel on a cache of about a gigabyte per layer (B sequences x ctx keys): the fixed costs of a call -- launch, first
    tile, read-out, merge -- weigh much less than on configuration 5's 130 MB per layer."""
    from qwen_tailor_b200.batch import attn_paged
    M, page = 4, 64
    per = (ctx + M + page - 1) // page
    n_pages = B * per + 1
    g, _ = rn_factory(torch, dev, 13)
    rn = lambda *s: torch.randn(s, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    layers = [dict(K=rn(n_pages, 2, page, 256), V=rn(n_pages, 2, page, 256), q=rn(B * M, 8, 256), k=rn(B * M, 2, 256), v=rn(B * M, 2, 256))
              for _ in range(n_layers)]
    bt = (1 + torch.arange(B * per, dtype=torch.int32, device=dev)).reshape(B, per).contiguous()
    cl = torch.full((B,), ctx, dtype=torch.int32, device=dev)

    def step():
        for L in layers:
            attn_paged(L["q"], L["k"], L["v"], L["K"], L["V"], bt, cl, M=M, max_ctx=ctx)

    ms = time_region(torch, graphed(torch, step), args.steps, repeats=3) / args.steps
    byts = n_layers * float(B * ctx) * 2048
    gbs = byts / (ms * 1e-3) / 1e9
    return dict(workload=f"GQA decode attention, B={B}, M=4, ctx={ctx}, {n_layers} layers, paged bf16 KV", ms_per_step=ms, kv_gb=byts / 1e9,
                roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"]))


def bench_prefill_attention(torch, dev, args, peaks, S=2048, n_layers=6):
    """Causal prefill attention of the full-attention layers (head_dim 256, 8 query heads on 2 KV heads): S tokens from position 0,
    n_layers layers with their own q / K / V.  FLOPs: 4 * 256 per (query head, query, visible key)."""
    from qwen_tailor_b200.attn_glue import prefill_attention
    g, _ = rn_factory(torch, dev, 17)
    rn = lambda *s: torch.randn(s, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    layers = [dict(q=rn(S, 8, 256), K=rn(2, S, 256), V=rn(2, S, 256)) for _ in range(n_layers)]

    def step():
        for L in layers:
            prefill_attention(L["q"], L["K"], L["V"], pos=0)

    ms = time_region(torch, graphed(torch, step), args.steps, repeats=3) / args.steps
    flops = n_layers * 4.0 * 256 * 8 * (S * (S + 1) / 2)
    tf = flops / (ms * 1e-3) / 1e12
    return dict(workload=f"causal prefill attention, S={S}, {n_layers} layers, 8 q heads / 2 KV heads, head_dim 256", ms_per_step=ms,
                tokens_per_s=S / (ms * 1e-3),
                roofline=dict(bound="tensor", achieved=tf, peak=peaks["bf16_tflops"], unit="TFLOP/s", frac=tf / peaks["bf16_tflops"]))


def bench_verify(torch, dev, args, peaks, n_layers=N_LAYERS, B=16):
    """Configuration 5, GDN part: B sequences x M=4 chained tokens through n_layers layers, per-token fp32 snapshots in place."""
    from qwen_tailor_b200.batch_spec import deltanet_bm
    M = 4
    g, _ = rn_factory(torch, dev, 11)
    layers = []
    for _ in range(n_layers):
        layers.append(dict(
            proj=torch.randn((B * M, PW), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16),
            conv=torch.randn(((B + 1) * 2, M, 3, CD), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16),
            conv_w=(torch.randn((CD * 4,), generator=g, device=dev, dtype=torch.float32) * 0.5).to(torch.bfloat16),
            A_log=torch.rand((HV,), generator=g, device=dev, dtype=torch.float32) * math.log(16.0),
            dt_bias=torch.zeros((HV,), device=dev, dtype=torch.float32),
            ssm=torch.randn((B + 1, M, HV, DV, DK), generator=g, device=dev, dtype=torch.float32) * 0.02))
    ss = torch.arange(B, dtype=torch.int32, device=dev)
    sels = torch.randint(0, M, (B,), generator=g, device=dev, dtype=torch.int32)
    pars = torch.zeros(B, dtype=torch.int32, device=dev)

    def step():
        for L in layers:
            deltanet_bm(L["proj"], L["conv"], L["conv_w"], L["A_log"], L["dt_bias"], L["ssm"], ss, sels, pars, M)

    ms = time_region(torch, graphed(torch, step), args.steps, repeats=3) / args.steps
    per = (1 + M) * STATE_BYTES + M * (CD * 2 + 3 * CD * 2 + HV * DV * 2) + 3 * CD * 2
    gbs = n_layers * B * per / (ms * 1e-3) / 1e9
    return dict(workload=f"GDN speculative verify, config 5 shape: B={B}, M=4, {n_layers} layers, snapshots [B,4,16,128,128] fp32 in place", ms_per_step=ms,
                roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"]))


def _prefill_inputs(torch, dev, g, total, n_groups=1):
    """q, k, v, log-decay, beta for `total` packed tokens (distributions of the benchmark configurations; one A_log per group)."""
    rn = lambda *s: torch.randn(s, generator=g, device=dev, dtype=torch.float32)
    unit = lambda x: x / x.norm(dim=-1, keepdim=True)
    q = (unit(rn(total, HV, DK)) * DK ** -0.5).to(torch.bfloat16)
    k = unit(rn(total, HV, DK)).to(torch.bfloat16)
    v = rn(total, HV, DV).to(torch.bfloat16)
    A = torch.exp(torch.rand((n_groups, 1, HV), generator=g, device=dev) * math.log(16.0))
    lg = (-A * torch.nn.functional.softplus(rn(n_groups, total // n_groups, HV))).reshape(total, HV).contiguous()
    beta = torch.sigmoid(rn(total, HV))
    return q, k, v, lg, beta


def _prefill_result(workload, ms, toks, n_states, peaks):
    tflops = toks * PREFILL_FLOP_PER_TOKEN_LAYER / (ms * 1e-3) / 1e12
    gbs = (toks * PREFILL_BYTES_PER_TOKEN_LAYER + n_states * STATE_BYTES) / (ms * 1e-3) / 1e9
    return dict(workload=workload, ms_per_step=ms, tokens_per_s=toks / (ms * 1e-3),
                roofline=dict(bound="tensor", achieved=tflops, peak=peaks["bf16_tflops"], unit="TFLOP/s", frac=tflops / peaks["bf16_tflops"]),
                hbm=dict(achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"]))


def bench_prefill(torch, dev, args, peaks, T=2048, n_layers=N_LAYERS, n_sets=3):
    """Configuration 3: one sequence of T tokens, chunk 64, applied as n_layers independent layers (one packed launch)."""
    from qwen_tailor_b200.gdn_nax import gdn_chunked_varlen
    g, _ = rn_factory(torch, dev, 100)
    n = n_layers
    sets = [_prefill_inputs(torch, dev, g, n * T, n_groups=n) for _ in range(n_sets)]     # rotated so that reads come from HBM
    cu = torch.arange(0, (n + 1) * T, T, dtype=torch.int32, device=dev)
    it = [0]

    def step():
        q, k, v, lg, beta = sets[it[0] % n_sets]
        it[0] += 1
        gdn_chunked_varlen(q, k, v, lg, beta, cu)

    for _ in range(3):
        step()
    ms = time_region(torch, step, args.steps, repeats=3) / args.steps
    return _prefill_result(f"GDN chunked prefill, config 3: B=1, T={T}, chunk 64, {n} independent layers, zero initial state", ms, n * T, n, peaks)


def config4_local(rank, world):
    """Suffix lengths and resume flags of this rank's sequences of benchmark configuration 4 (greedy split by token count)."""
    import numpy as np
    from qwen_tailor_b200 import synth
    from qwen_tailor_b200.shard import partition_sequences
    lengths, prefix = synth.config4_lengths()
    suffix = (lengths - prefix).astype(np.int64)
    parts = partition_sequences([int(x) for x in suffix], world)
    loads = [int(sum(suffix[i] for i in p)) for p in parts]
    mine = parts[rank]
    return suffix[mine], (prefix[mine] > 0), loads, int(suffix.sum())


def bench_prefill_ragged(torch, dev, args, peaks, dist=None, n_layers=6):
    """Configuration 4: 16 sequences ~U[128, 4096] packed by cu_seqlens, every second one resuming from a cached fp32 state at a
    64-aligned prefix (only the suffix is computed); n_layers independent layers per launch.  With several ranks the sequences are
    sharded by token count (no collective) and the same batch is timed: strong scaling."""
    import numpy as np
    from qwen_tailor_b200.gdn_nax import gdn_chunked_varlen
    rank, world = (dist.get_rank(), dist.get_world_size()) if dist is not None else (0, 1)
    suffix, resumes, loads, total_all = config4_local(rank, world)
    n_seq = len(suffix)
    cu = np.zeros(n_layers * n_seq + 1, np.int64)
    cu[1:] = np.cumsum(np.tile(suffix, n_layers))
    total = int(cu[-1])
    g, rn = rn_factory(torch, dev, 7 + rank)
    q, k, v, lg, beta = _prefill_inputs(torch, dev, g, max(total, 1))
    init = rn(max(n_seq, 1), HV, DV, DK) * 0.02
    idx = torch.tensor(np.tile(np.where(resumes, np.arange(n_seq), -1), n_layers), dtype=torch.int32, device=dev)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)

    def step():
        if n_seq:
            gdn_chunked_varlen(q[:total], k[:total], v[:total], lg[:total], beta[:total], cu_t, init_state=init, init_idx=idx)

    for _ in range(3):
        step()
    ms = time_region(torch, step, args.steps, dist, repeats=3) / args.steps
    toks = total_all * n_layers
    out = _prefill_result(f"GDN ragged prefill, config 4: 16 sequences ~U[128,4096] with prefix resume, {n_layers} layers per launch, "
                          f"sequences sharded over {world} GPU(s)", ms, toks, 16 * n_layers, peaks)
    out["scaling"] = "strong"
    out["tokens_per_rank"] = loads
    out["load_max_over_mean"] = max(loads) / (sum(loads) / len(loads))
    # the tensor roofline of N GPUs is N times the peak of one
    out["roofline"]["peak"] *= world
    out["roofline"]["frac"] /= world
    out["hbm"]["peak"] *= world
    out["hbm"]["frac"] /= world
    return out


def bench_prefill_single(torch, dev, args, peaks, dist=None, T=8192):
    """Configuration 3, one layer of one sequence of T tokens.  With several ranks the 16 heads are split over the ranks and y is
    all-gathered over NCCL (strong scaling)."""
    from qwen_tailor_b200.shard import prefill_head_sharded
    rank, world = (dist.get_rank(), dist.get_world_size()) if dist is not None else (0, 1)
    g, _ = rn_factory(torch, dev, 100)
    q, k, v, lg, beta = _prefill_inputs(torch, dev, g, T)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)

    def step():
        prefill_head_sharded(q, k, v, lg, beta, cu, rank, world)

    for _ in range(3):
        step()
    ms = time_region(torch, step, args.steps, dist, repeats=3) / args.steps
    out = _prefill_result(f"GDN prefill, config 3: one layer of one sequence, T={T}, 16 heads over {world} GPU(s)"
                          + (", NCCL all-gather of y" if world > 1 else ""), ms, T, 1, peaks)
    out["scaling"] = "strong"
    out["roofline"]["peak"] *= world
    out["roofline"]["frac"] /= world
    out["hbm"]["peak"] *= world
    out["hbm"]["frac"] /= world
    return out


# ----------------------------------------------------------------------------------------------------------------------
# CPU baseline (OpenMP C port of the reference's arithmetic; test infrastructure, timed only)
# ----------------------------------------------------------------------------------------------------------------------
def cpu_decode_steps(n_steps, warmup, B=B_DECODE, n_layers=N_LAYERS):
    import numpy as np
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU baseline is meant to use every host core
    os.environ["OMP_NUM_THREADS"] = os.environ.get("GDN_CPU_THREADS", str(os.cpu_count() or 1))
    from oracle import build_oracle as co
    rng = np.random.default_rng(1)
    bits = lambda x: (x.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    layers = []
    for _ in range(n_layers):
        layers.append(dict(proj=bits(rng.standard_normal((B, PW))), conv=bits(rng.standard_normal(((B + 1) * 2, 3, CD))),
                           ssm=(rng.standard_normal((B + 1, HV, DV, DK)) * 0.02).astype(np.float32)))
    A_log = rng.uniform(0, math.log(16.0), HV).astype(np.float32)
    dtb = np.zeros(HV, np.float32)
    slots = np.arange(B, dtype=np.int32)
    pos = np.zeros(B, np.int32)
    conv_w = bits(rng.standard_normal(CD * 4))

    def step():
        for L in layers:
            co.deltanet_b(L["proj"], L["conv"], conv_w, A_log, dtb, L["ssm"], slots, pos)
        pos[:] += 1

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(n_steps):
        step()
    dt = time.perf_counter() - t0
    return n_steps / dt, dt / n_steps * 1e3, co.max_threads()


def run_reference(args):
    """The reference arm: the CPU restatement of the decode step on all host cores (the reference's own code is Metal-only and has
    no C sources to build).  A full step takes ~35 ms on 16 cores, so K steps after W warm-up steps stay within seconds."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    v, ms, cores = cpu_decode_steps(args.steps, args.warmup)
    line = dict(metric="gdn_decode_steps_per_s_B64", value=v, unit="steps/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=config_block(args.gpus),
                cpu_baseline=dict(value=v, unit="steps/s", cores=cores, kind="port",
                                  sample=f"{args.steps} full steps (64 sequences x 18 layers each) after {args.warmup} warm-up steps, "
                                         "OpenMP C port of the reference's decode arithmetic"),
                e2e=dict(value=v, unit="steps/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


def config_block(n_gpus):
    return dict(workload="configs[1]: GDN recurrent decode step, B=64 sequences per GPU, 18 GatedDeltaNet layers per step "
                         "(conv1d k=4 on mixed qkv 6144 + l2norm + gates + delta rule, fp32 state [16,128,128], in-place slot pools)",
                batch_per_gpu=B_DECODE, layers=N_LAYERS, parallelism=f"sequence-sharded x{n_gpus} (no collective)",
                l2_policy="inputs larger than L2: 18 per-layer state pools (1.2 GB) are cycled through every step")


# ----------------------------------------------------------------------------------------------------------------------
# the additional workloads: each one is timed on its own, its failure is recorded instead of raised, and the device status word
# is read (and cleared) after every one of them
# ----------------------------------------------------------------------------------------------------------------------
def run_extras(torch, dev, args, peaks, _lib, dist=None):
    a2 = copy.copy(args)
    a2.steps = max(5, args.steps // 2)
    world = dist.get_world_size() if dist is not None else 1
    if world == 1:
        def dec(B):
            d = bench_decode(torch, dev, a2, None, peaks, B=B, with_e2e=False)
            return dict(steps_per_s=1e3 / d["ms_per_step"], launch_us=d["launch_us"], hbm_gbs=d["achieved_gbs"], frac=d["frac"])
        legs = [("decode_B1", lambda: dec(1)), ("decode_B16", lambda: dec(16)),
                ("verify_config5", lambda: bench_verify(torch, dev, a2, peaks)),
                ("verify_B64_M4", lambda: bench_verify(torch, dev, a2, peaks, n_layers=6, B=64)),
                ("attention_config5", lambda: bench_attention(torch, dev, a2, peaks)),
                ("attention_B64_ctx8192", lambda: bench_attention_large(torch, dev, a2, peaks)),
                ("prefill_attention_S2048", lambda: bench_prefill_attention(torch, dev, a2, peaks)),
                ("prefill_attention_S8192", lambda: bench_prefill_attention(torch, dev, a2, peaks, S=8192)),
                ("prefill_T2048", lambda: bench_prefill(torch, dev, a2, peaks)),
                ("prefill_T8192", lambda: bench_prefill(torch, dev, a2, peaks, T=8192, n_layers=9, n_sets=2)),
                ("prefill_T8192_one_sequence", lambda: bench_prefill_single(torch, dev, a2, peaks)),
                ("prefill_ragged_config4", lambda: bench_prefill_ragged(torch, dev, a2, peaks))]
    else:
        legs = [("prefill_T8192_head_sharded", lambda: bench_prefill_single(torch, dev, a2, peaks, dist)),
                ("prefill_ragged_config4_sharded", lambda: bench_prefill_ragged(torch, dev, a2, peaks, dist))]
    only = set(args.only.split(",")) if getattr(args, "only", None) else None
    extra = {}
    for name, fn in legs:
        if only is not None and name not in only:
            continue
        try:
            res = fn()
        except Exception as e:                              # recorded, never raised: the other workloads still run
            res = dict(error=f"{type(e).__name__}: {e}", trace=traceback.format_exc(limit=3))
        try:
            st = read_status(_lib)
        except Exception as e:
            st = dict(code=None, meaning=f"status unreadable: {e}")
        if dist is not None:                                # every rank's word counts
            t = torch.tensor([st["code"] if st["code"] is not None else -1], dtype=torch.int32, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            code = int(t.item())
            st = dict(code=code, meaning=STATUS_NAMES.get(code, "unknown"))
        if isinstance(res, dict):
            res["device_status"] = st
        extra[name] = res
    return extra


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the additional workloads (prefill, verify, attention, small batches)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--extras-child", action="store_true", help="run only the additional single-GPU workloads and print them as one JSON object")
    ap.add_argument("--only", default=None, help="comma-separated names of the additional workloads to run (with --extras-child)")
    ap.add_argument("--case", default=None, choices=["prefill", "attention", "verify", "decode", "prefill_attention"],
                    help="run only this small workload a few times and print its line (used for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    from qwen_tailor_b200 import _lib
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from qwen_tailor_b200.shard import bind_host_to_gpu
    host_binding = bind_host_to_gpu(local)               # pinned buffers of this rank then lie in the GPU's own NUMA node
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    peaks = measured_peaks()

    if args.case:
        a2 = argparse.Namespace(steps=max(1, min(args.steps, 3)), warmup=3)
        if args.case == "prefill":
            out = bench_prefill(torch, dev, a2, peaks, n_layers=9, n_sets=1)     # 9 x 16 chains = one wave of 144 blocks, 0.3 GB of inputs
        elif args.case == "attention":
            out = bench_attention(torch, dev, a2, peaks, n_layers=2)
        elif args.case == "prefill_attention":
            out = bench_prefill_attention(torch, dev, a2, peaks, S=4096, n_layers=1)
        elif args.case == "decode":
            d = bench_decode(torch, dev, a2, None, peaks, n_layers=4, with_e2e=False)
            out = dict(launch_us=d["launch_us"], hbm_gbs=d["achieved_gbs"], frac=d["frac"])
        else:
            out = [bench_verify(torch, dev, a2, peaks, n_layers=4), bench_verify(torch, dev, a2, peaks, n_layers=4, B=64)]
        print(json.dumps(dict(result=out, device_status=read_status(_lib))))
        return

    if args.extras_child:
        print(json.dumps(run_extras(torch, dev, args, peaks, _lib)))
        return

    sampler = ClockSampler(local)
    sampler.start()
    dec = bench_decode(torch, dev, args, dist, peaks)
    clocks = sampler.stop()
    status = read_status(_lib)

    n = world
    value = n * 1e3 / dec["ms_per_step"]
    line = dict(metric="gdn_decode_steps_per_s_B64", value=value, unit="steps/s", n_gpus=n, steps=args.steps, warmup=args.warmup,
                ms_per_step=dec["ms_per_step"], higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                config=config_block(n), clocks=clocks, gpu_launches=dec["launches"], timed_regions=REGION_REPEATS,
                layer_steps_per_s=value * N_LAYERS, sequence_tokens_per_s=value * B_DECODE,
                e2e=dict(value=n * 1e3 / dec["e2e_ms_per_step"], unit="steps/s", h2d_bytes_per_step=dec["h2d"], d2h_bytes_per_step=dec["d2h"]),
                roofline=dict(bound="hbm", kernel="gdn_decode_kernel<1>", achieved=dec["achieved_gbs"], peak=peaks["hbm_gbs"], unit="GB/s",
                              frac=dec["frac"], peak_source=peaks["source"], launch_us=dec["launch_us"],
                              algorithmic_bytes_per_launch=B_DECODE * DECODE_BYTES_PER_SEQ_LAYER, traffic=DECODE_TRAFFIC_NCU),
                device_status=status, host_binding=host_binding)
    if not args.no_extra:
        if world == 1:
            # in a child process: whatever happens there, the headline above survives
            cmd = [sys.executable, str(Path(__file__).resolve()), "--extras-child", "--steps", str(args.steps), "--warmup", str(args.warmup)]
            try:
                p = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
                last = [ln for ln in p.stdout.strip().splitlines() if ln.startswith("{")]
                line["extra"] = json.loads(last[-1]) if last else dict(error=f"child exited {p.returncode}", stderr=p.stderr[-800:])
            except Exception as e:
                line["extra"] = dict(error=f"{type(e).__name__}: {e}")
        else:
            try:
                extra = run_extras(torch, dev, args, peaks, _lib, dist)
            except Exception as e:
                extra = dict(error=f"{type(e).__name__}: {e}")
            line["extra"] = extra
    if rank == 0 and not args.no_cpu:
        try:
            v, ms, cores = cpu_decode_steps(3, 1)
            line["cpu_baseline"] = dict(value=v, unit="steps/s", cores=cores, kind="port",
                                        sample="3 full steps (64 sequences x 18 layers each) after 1 warm-up, OpenMP C port of the reference's decode arithmetic")
        except Exception as e:
            line["cpu_baseline"] = dict(value=None, unit="steps/s", cores=0, kind="port", sample=f"failed: {e}")
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
