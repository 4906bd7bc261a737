"""Benchmark of the GatedDeltaNet / GQA-decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Headline line (one JSON object on stdout, rank 0):
  metric   decode steps/s at B=64 -- one step = one token for each of 64 sequences through the model's 18 GatedDeltaNet layers
           (benchmark configuration 2: conv1d k=4 over the mixed qkv row, q/k l2norm, gates, gated delta rule on the fp32
           [16,128,128] state, in-place slot pools).  With N GPUs the batch is sharded by sequence: every GPU owns its own 64
           sequences (weak scaling, no collective on the data path) and `value` is the sum over GPUs.
  value    kernel-only throughput, state pools and inputs resident in HBM, the 18 launches of a step replayed from a CUDA graph.
  e2e      the same step through the Python operator API with the step's inputs (proj rows) in pinned host memory and the outputs
           read back to the host inside the timed region.
  roofline HBM roofline of the decode kernel: algorithmic bytes per launch / average launch time, against the measured copy bandwidth.
  extra    further workloads of the hot path measured in the same run (chunked prefill at T=2048 x 18 layers, speculative verify
           + paged GQA attention of configuration 5, decode at B=1/16), each with its own roofline fraction.
`--impl reference` times the CPU restatement of the reference's arithmetic (OpenMP C port, all host threads) on the same step.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
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
# dram__bytes_read.sum + dram__bytes_write.sum of one decode launch at B=64 from the ncu capture summarised in
# profiles/gdn_decode_kernel_B64.md (70.34 MB read + 12.64 MB written; the rest of the 67 MB of state written by a launch is
# still in L2 when the kernel ends and is written back during the following launches)
DECODE_TRAFFIC_NCU = 82978816
PREFILL_FLOP_PER_TOKEN_LAYER = HV * (8 * 64 * 128 + 6 * 128 * 128)        # chunk 64: 2,621,440
PREFILL_BYTES_PER_TOKEN_LAYER = 4 * HV * 128 * 2 + 2 * HV * 4                # q,k,v,y bf16 + log-decay, beta fp32 = 16,512


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


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
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
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
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "power_w_max": max(power) if power else None}


# ----------------------------------------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------------------------------------
def make_decode_layers(torch, dev, B, n_layers, seed):
    """Per-layer slot pools and inputs of benchmark configuration 2 (state ~ N(0, 0.02), everything else ~ N(0, 1))."""
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    layers = []
    for _ in range(n_layers):
        L = dict(
            proj=torch.randn((B, PW), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16),
            conv_pool=torch.randn(((B + 1) * 2, 3, CD), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16),
            conv_w=(torch.randn((CD * 4,), generator=g, device=dev, dtype=torch.float32) * 0.5).to(torch.bfloat16),
            A_log=torch.rand((HV,), generator=g, device=dev, dtype=torch.float32) * math.log(16.0),
            dt_bias=(torch.randn((HV,), generator=g, device=dev, dtype=torch.float32) * 0.1).to(torch.bfloat16).float(),
            ssm_pool=torch.randn((B + 1, HV, DV, DK), generator=g, device=dev, dtype=torch.float32) * 0.02,
        )
        layers.append(L)
    return layers


def time_region(torch, fn, iters, dist=None):
    """Run fn() `iters` times between CUDA events on the current stream, bracketed by barrier + synchronize.  Returns ms (max over ranks)."""
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    return ms


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


def bench_decode(torch, dev, args, dist, peaks, B=B_DECODE, n_layers=N_LAYERS, with_e2e=True):
    from qwen_tailor_b200.batch import deltanet_b
    layers = make_decode_layers(torch, dev, B, n_layers, seed=1 + (dist.get_rank() if dist else 0))
    slots = torch.arange(B, dtype=torch.int32, device=dev)
    pos = torch.zeros(B, dtype=torch.int32, device=dev)
    ys = [None] * n_layers

    def step():
        for i, L in enumerate(layers):
            ys[i] = deltanet_b(L["proj"], L["conv_pool"], L["conv_w"], L["A_log"], L["dt_bias"], L["ssm_pool"], slots, pos)
        pos.add_(1)                                       # flips the conv double buffer like a real decode loop

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    ms = time_region(torch, graph.replay, args.steps, dist)
    ms_per_step = ms / args.steps
    launch_us = ms_per_step * 1e3 / n_layers
    gbs = B * DECODE_BYTES_PER_SEQ_LAYER / (launch_us * 1e-6) / 1e9
    out = dict(ms_per_step=ms_per_step, launch_us=launch_us, achieved_gbs=gbs, frac=gbs / peaks["hbm_gbs"], launches=args.steps * n_layers,
               state_gb=n_layers * (B + 1) * STATE_BYTES / 1e9)
    if with_e2e:
        host_proj = [torch.randn((B, PW), dtype=torch.float32).to(torch.bfloat16).pin_memory() for _ in range(n_layers)]
        host_y = [torch.empty((B, HV * DV), dtype=torch.bfloat16).pin_memory() for _ in range(n_layers)]

        def e2e_step():
            for i, L in enumerate(layers):
                L["proj"].copy_(host_proj[i], non_blocking=True)
            graph.replay()                                # the 18 operator calls of a step, captured once (as the reference compiles its step)
            for i in range(n_layers):
                host_y[i].copy_(ys[i], non_blocking=True)
            torch.cuda.current_stream().synchronize()     # the caller reads the step's result before launching the next one

        for _ in range(3):
            e2e_step()
        ms_e = time_region(torch, e2e_step, args.steps, dist)
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
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    rn = lambda *s: torch.randn(s, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    layers = [dict(K=rn(n_pages, 2, page, 256), V=rn(n_pages, 2, page, 256), q=rn(B * M, 8, 256), k=rn(B * M, 2, 256), v=rn(B * M, 2, 256))
              for _ in range(n_layers)]
    bt = torch.from_numpy(table).to(dev)
    cl = torch.from_numpy(ctx).to(dev)
    mc = int(ctx.max())

    def step():
        for L in layers:
            attn_paged(L["q"], L["k"], L["v"], L["K"], L["V"], bt, cl, M=M, max_ctx=mc)

    ms = time_region(torch, graphed(torch, step), args.steps) / args.steps
    byts = n_layers * float(ctx.sum()) * 2048
    gbs = byts / (ms * 1e-3) / 1e9
    return dict(workload=f"GQA decode attention, config 5: B=16, M=4, {n_layers} layers, paged bf16 KV, ctx~U[1024,8192]", ms_per_step=ms,
                kv_gb=byts / 1e9, roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"]))


def bench_verify(torch, dev, args, peaks, n_layers=N_LAYERS, B=16):
    """Configuration 5, GDN part: B sequences x M=4 chained tokens through n_layers layers, per-token fp32 snapshots in place."""
    from qwen_tailor_b200.batch_spec import deltanet_bm
    M = 4
    g = torch.Generator(device=dev)
    g.manual_seed(11)
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

    ms = time_region(torch, graphed(torch, step), args.steps) / args.steps
    per = (1 + M) * STATE_BYTES + M * (CD * 2 + 3 * CD * 2 + HV * DV * 2) + 3 * CD * 2
    gbs = n_layers * B * per / (ms * 1e-3) / 1e9
    return dict(workload=f"GDN speculative verify, config 5 shape: B={B}, M=4, {n_layers} layers, snapshots [B,4,16,128,128] fp32 in place", ms_per_step=ms,
                roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"]))


def bench_prefill(torch, dev, args, peaks, T=2048, n_layers=N_LAYERS):
    """Configuration 3: one sequence of T tokens, chunk 64, applied as 18 independent layers (one packed launch)."""
    try:
        from qwen_tailor_b200.gdn_nax import gdn_chunked_varlen
    except ImportError:
        return None
    g = torch.Generator(device=dev)
    g.manual_seed(100)
    n = n_layers
    rn = lambda *s: torch.randn(s, generator=g, device=dev, dtype=torch.float32)
    unit = lambda x: x / x.norm(dim=-1, keepdim=True)
    sets = []
    for _ in range(3):                                                 # rotate 3 input sets (3 x 0.6 GB) so that reads come from HBM
        q = (unit(rn(n * T, HV, DK)) * DK ** -0.5).to(torch.bfloat16)
        k = unit(rn(n * T, HV, DK)).to(torch.bfloat16)
        v = rn(n * T, HV, DV).to(torch.bfloat16)
        A = torch.exp(torch.rand((n, 1, HV), generator=g, device=dev) * math.log(16.0))
        lg = (-A * torch.nn.functional.softplus(rn(n, T, HV))).reshape(n * T, HV).contiguous()
        beta = torch.sigmoid(rn(n * T, HV))
        sets.append((q, k, v, lg, beta))
    cu = torch.arange(0, (n + 1) * T, T, dtype=torch.int32, device=dev)
    it = [0]

    def step():
        q, k, v, lg, beta = sets[it[0] % 3]
        it[0] += 1
        gdn_chunked_varlen(q, k, v, lg, beta, cu)

    for _ in range(3):
        step()
    ms = time_region(torch, step, args.steps) / args.steps
    toks = n * T
    tflops = toks * PREFILL_FLOP_PER_TOKEN_LAYER / (ms * 1e-3) / 1e12
    gbs = (toks * PREFILL_BYTES_PER_TOKEN_LAYER + n * STATE_BYTES) / (ms * 1e-3) / 1e9
    return dict(workload=f"GDN chunked prefill, config 3: B=1, T={T}, chunk 64, {n} independent layers, zero initial state", ms_per_step=ms,
                tokens_per_s=toks / (ms * 1e-3),
                roofline=dict(bound="tensor", achieved=tflops, peak=peaks["bf16_tflops"], unit="TFLOP/s", frac=tflops / peaks["bf16_tflops"]),
                hbm=dict(achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"]))


def bench_prefill_ragged(torch, dev, args, peaks, n_layers=6):
    """Configuration 4: 16 sequences ~U[128, 4096] packed by cu_seqlens, every second one resuming from a cached fp32 state at a
    64-aligned prefix (only the suffix is computed); here n_layers independent layers per launch."""
    import numpy as np
    from qwen_tailor_b200 import synth
    from qwen_tailor_b200.gdn_nax import gdn_chunked_varlen
    lengths, prefix = synth.config4_lengths()
    suffix = (lengths - prefix).astype(np.int64)
    n_seq = len(suffix)
    cu = np.zeros(n_layers * n_seq + 1, np.int64)
    cu[1:] = np.cumsum(np.tile(suffix, n_layers))
    total = int(cu[-1])
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    rn = lambda *s: torch.randn(s, generator=g, device=dev, dtype=torch.float32)
    unit = lambda x: x / x.norm(dim=-1, keepdim=True)
    q = (unit(rn(total, HV, DK)) * DK ** -0.5).to(torch.bfloat16)
    k = unit(rn(total, HV, DK)).to(torch.bfloat16)
    v = rn(total, HV, DV).to(torch.bfloat16)
    lg = -torch.exp(torch.rand((1, HV), generator=g, device=dev) * math.log(16.0)) * torch.nn.functional.softplus(rn(total, HV))
    beta = torch.sigmoid(rn(total, HV))
    init = rn(n_seq, HV, DV, DK) * 0.02
    idx = torch.tensor(np.tile(np.where(prefix > 0, np.arange(n_seq), -1), n_layers), dtype=torch.int32, device=dev)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)

    def step():
        gdn_chunked_varlen(q, k, v, lg.contiguous(), beta, cu_t, init_state=init, init_idx=idx)

    for _ in range(3):
        step()
    ms = time_region(torch, step, args.steps) / args.steps
    tflops = total * PREFILL_FLOP_PER_TOKEN_LAYER / (ms * 1e-3) / 1e12
    return dict(workload=f"GDN ragged prefill, config 4: 16 sequences ~U[128,4096] with prefix resume, {n_layers} layers per launch", ms_per_step=ms,
                tokens_per_s=total / (ms * 1e-3), roofline=dict(bound="tensor", achieved=tflops, peak=peaks["bf16_tflops"], unit="TFLOP/s",
                                                                frac=tflops / peaks["bf16_tflops"]))


def bench_prefill_head_sharded(torch, dev, args, dist, peaks, T=8192):
    """Configuration 3, head-parallel: one sequence of T tokens, the 16 heads split over the ranks, y all-gathered over NCCL."""
    from qwen_tailor_b200.shard import prefill_head_sharded
    world, rank = dist.get_world_size(), dist.get_rank()
    g = torch.Generator(device=dev)
    g.manual_seed(100)
    rn = lambda *s: torch.randn(s, generator=g, device=dev, dtype=torch.float32)
    unit = lambda x: x / x.norm(dim=-1, keepdim=True)
    q = (unit(rn(T, HV, DK)) * DK ** -0.5).to(torch.bfloat16)
    k = unit(rn(T, HV, DK)).to(torch.bfloat16)
    v = rn(T, HV, DV).to(torch.bfloat16)
    lg = (-torch.exp(torch.rand((1, HV), generator=g, device=dev) * math.log(16.0)) * torch.nn.functional.softplus(rn(T, HV))).contiguous()
    beta = torch.sigmoid(rn(T, HV))
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)

    def step():
        prefill_head_sharded(q, k, v, lg, beta, cu, rank, world)

    for _ in range(3):
        step()
    ms = time_region(torch, step, args.steps, dist) / args.steps
    return dict(workload=f"GDN prefill, config 3 head-parallel: B=1, T={T}, 16 heads over {world} GPUs, NCCL all-gather of y", ms_per_step=ms,
                tokens_per_s=T / (ms * 1e-3))


# ----------------------------------------------------------------------------------------------------------------------
# CPU baseline (OpenMP C port of the reference's arithmetic; test infrastructure, timed only)
# ----------------------------------------------------------------------------------------------------------------------
def cpu_decode_steps(n_steps, warmup, B=B_DECODE, n_layers=N_LAYERS):
    import numpy as np
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU baseline is meant to use every host core
    os.environ["OMP_NUM_THREADS"] = os.environ.get("GDN_CPU_THREADS", str(os.cpu_count() or 1))
    from oracle import build_oracle as co
    rng = np.random.default_rng(1)
    conv_w = (rng.integers(0, 1 << 15, CD * 4)).astype(np.uint16)
    layers = []
    for _ in range(n_layers):
        layers.append(dict(proj=(rng.standard_normal((B, PW)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16),
                           conv=(rng.standard_normal(((B + 1) * 2, 3, CD)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16),
                           ssm=(rng.standard_normal((B + 1, HV, DV, DK)) * 0.02).astype(np.float32)))
    A_log = rng.uniform(0, math.log(16.0), HV).astype(np.float32)
    dtb = np.zeros(HV, np.float32)
    slots = np.arange(B, dtype=np.int32)
    pos = np.zeros(B, np.int32)
    conv_w = (rng.standard_normal(CD * 4).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)

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
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = min(args.steps, 20)
    v, ms, cores = cpu_decode_steps(steps, min(args.warmup, 3))
    line = dict(metric="gdn_decode_steps_per_s_B64", value=v, unit="steps/s", n_gpus=args.gpus, steps=steps, warmup=min(args.warmup, 3),
                ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=config_block(args.gpus),
                cpu_baseline=dict(value=v, unit="steps/s", cores=cores, kind="port",
                                  sample=f"{steps} full steps (64 sequences x 18 layers each), OpenMP C port of the reference's decode arithmetic"),
                e2e=dict(value=v, unit="steps/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


def config_block(n_gpus):
    return dict(workload="configs[1]: GDN recurrent decode step, B=64 sequences per GPU, 18 GatedDeltaNet layers per step "
                         "(conv1d k=4 on mixed qkv 6144 + l2norm + gates + delta rule, fp32 state [16,128,128], in-place slot pools)",
                batch_per_gpu=B_DECODE, layers=N_LAYERS, parallelism=f"sequence-sharded x{n_gpus} (no collective)",
                l2_policy="inputs larger than L2: 18 per-layer state pools (1.2 GB) are cycled through every step")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the additional workloads (prefill, verify, attention, small batches)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--case", default=None, choices=["prefill", "attention", "verify"],
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
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    peaks = measured_peaks()

    if args.case:
        a2 = argparse.Namespace(steps=max(1, min(args.steps, 3)), warmup=3)
        if args.case == "prefill":
            out = bench_prefill(torch, dev, a2, peaks, n_layers=9)       # 9 x 16 chains = one wave of 144 blocks, 0.3 GB of inputs
        elif args.case == "attention":
            out = bench_attention(torch, dev, a2, peaks, n_layers=2)
        else:
            out = [bench_verify(torch, dev, a2, peaks, n_layers=4), bench_verify(torch, dev, a2, peaks, n_layers=4, B=64)]
        print(json.dumps(out))
        return

    sampler = ClockSampler(local)
    sampler.start()
    dec = bench_decode(torch, dev, args, dist, peaks)
    clocks = sampler.stop()

    n = world
    value = n * 1e3 / dec["ms_per_step"]
    line = dict(metric="gdn_decode_steps_per_s_B64", value=value, unit="steps/s", n_gpus=n, steps=args.steps, warmup=args.warmup,
                ms_per_step=dec["ms_per_step"], higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                config=config_block(n), clocks=clocks, gpu_launches=dec["launches"],
                layer_steps_per_s=value * N_LAYERS, sequence_tokens_per_s=value * B_DECODE,
                e2e=dict(value=n * 1e3 / dec["e2e_ms_per_step"], unit="steps/s", h2d_bytes_per_step=dec["h2d"], d2h_bytes_per_step=dec["d2h"]),
                roofline=dict(bound="hbm", kernel="gdn_decode_kernel<2>", achieved=dec["achieved_gbs"], peak=peaks["hbm_gbs"], unit="GB/s",
                              frac=dec["frac"], peak_source=peaks["source"], launch_us=dec["launch_us"],
                              algorithmic_bytes_per_launch=B_DECODE * DECODE_BYTES_PER_SEQ_LAYER, traffic=DECODE_TRAFFIC_NCU))
    if rank == 0 and world == 1:
        extra = {}
        if not args.no_extra:
            import copy
            a2 = copy.copy(args)
            a2.steps = max(10, args.steps // 2)
            for B in (1, 16):
                d = bench_decode(torch, dev, a2, None, peaks, B=B, with_e2e=False)
                extra[f"decode_B{B}"] = dict(steps_per_s=1e3 / d["ms_per_step"], launch_us=d["launch_us"], hbm_gbs=d["achieved_gbs"], frac=d["frac"])
            extra["verify_config5"] = bench_verify(torch, dev, a2, peaks)
            extra["verify_B64_M4"] = bench_verify(torch, dev, a2, peaks, n_layers=6, B=64)
            extra["attention_config5"] = bench_attention(torch, dev, a2, peaks)
            p = bench_prefill(torch, dev, a2, peaks)
            if p is not None:
                extra["prefill_T2048"] = p
                extra["prefill_T8192"] = bench_prefill(torch, dev, a2, peaks, T=8192, n_layers=9)
                extra["prefill_ragged_config4"] = bench_prefill_ragged(torch, dev, a2, peaks)
        line["extra"] = extra
        if not args.no_cpu:
            v, ms, cores = cpu_decode_steps(3, 1)
            line["cpu_baseline"] = dict(value=v, unit="steps/s", cores=cores, kind="port",
                                        sample="3 full steps (64 sequences x 18 layers each) after 1 warm-up, OpenMP C port of the reference's decode arithmetic")
        assert _lib.device_status() == 0, "a kernel reported an out-of-range index"
    if world > 1 and not args.no_extra:
        import copy
        a3 = copy.copy(args)
        a3.steps = max(5, args.steps // 4)
        hs = bench_prefill_head_sharded(torch, dev, a3, dist, peaks)
        if rank == 0:
            line["extra"] = {"prefill_T8192_head_sharded": hs}
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
