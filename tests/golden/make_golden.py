"""Generate tests/golden/rec64_kat.npz by running the reference's own CPU statement of the gated delta rule.

The reference's only host-executable code for this path is ``rec64`` in ``bench/gdn_f64.py:48-56`` (numpy fp64).  The file
around it imports MLX and loads model weights at import time, so this script does not import it: it parses the file, takes
the ``rec64`` function definition unmodified out of the syntax tree and executes only that definition with numpy in scope.
Inputs are seeded bf16-exact arrays with the value distributions of the benchmark configurations; they are stored next to
the outputs so the fixture does not depend on a random-number implementation (the initial state is a closed-form array).

Run (needs the reference checkout):  python tests/golden/make_golden.py /path/to/reference
"""
import ast
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from qwen_tailor_b200 import synth                      # noqa: E402
from oracle import gdn_oracle as orc                    # noqa: E402


def reference_rec64(ref_root: Path):
    src = (ref_root / "bench" / "gdn_f64.py").read_text()
    tree = ast.parse(src)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "rec64")
    mod = ast.Module(body=[fn], type_ignores=[])
    ns = {"np": np}
    exec(compile(mod, "gdn_f64.py:rec64", "exec"), ns)
    return ns["rec64"]


def warm_state(scale):
    """Closed-form initial state (no random numbers): scale * cos(0.37 h + 0.11 v + 0.05 k + 0.013 v k), fp32 [16,128,128]."""
    h = np.arange(16)[:, None, None]
    v = np.arange(128)[None, :, None]
    k = np.arange(128)[None, None, :]
    return (scale * np.cos(0.37 * h + 0.11 * v + 0.05 * k + 0.013 * v * k)).astype(np.float32)


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path of a checkout of the reference project>")
    ref_root = Path(sys.argv[1])
    rec64 = reference_rec64(ref_root)
    out = {}
    for name, T, seed, state_scale in (("zero_state", 24, 0, 0.0), ("warm_state", 17, 1, 0.02)):
        rng = np.random.default_rng(seed)
        A_log, dt_bias = synth.layer_params(rng)
        q, k, v, a, b = synth.gdn_tokens(rng, T)
        g = orc.compute_g(A_log, a, dt_bias).astype(np.float64)
        beta = orc.beta_gate(b).astype(np.float64)
        S0 = warm_state(state_scale).astype(np.float64)
        y, S = rec64(q.astype(np.float64), k.astype(np.float64), v.astype(np.float64), g, beta, S0)
        out[f"{name}_q"] = orc.bf16_bits(q)
        out[f"{name}_k"] = orc.bf16_bits(k)
        out[f"{name}_v"] = orc.bf16_bits(v)
        out[f"{name}_g"] = g
        out[f"{name}_beta"] = beta.astype(np.float32)
        out[f"{name}_state_scale"] = np.array([state_scale])
        out[f"{name}_y"] = y.astype(np.float32)                   # [T,16,128]
        out[f"{name}_y_sum"] = y.sum(axis=2)                      # fp64 checksums per (token, head)
        out[f"{name}_S_rows"] = S[:, ::16, :].astype(np.float32)  # every 16th value row of the final state
        out[f"{name}_S_sum"] = S.sum(axis=2)                      # fp64 checksum of every state row
    np.savez_compressed(Path(__file__).with_name("rec64_kat.npz"), **out)
    print("wrote", Path(__file__).with_name("rec64_kat.npz"))


if __name__ == "__main__":
    main()
