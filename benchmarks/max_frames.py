"""Largest trainable frame count at a given resolution and layout, found without ever running out of memory.

Peak memory of a training step is affine in the number of latent frames (weights, gradients and optimizer state are
fixed; activations, attention workspaces and saved attention outputs grow with the token count).  The tool measures
the peak at two small frame counts with ``bench.py``, fits the line, proposes the largest ``4k + 1`` frame count whose
predicted peak stays below ``--limit-gb``, and (unless ``--no-verify``) runs that one once to confirm.  It never probes
upwards until something fails: a run that exhausted device memory could take the machine down for other users.

    python benchmarks/max_frames.py --gpus 8 --tp 1 --cp 8 --limit-gb 165

Every measurement is one ``bench.py`` launch (``torch.distributed.run`` for more than one GPU) with one warm-up and one
timed step; the JSON line that ``bench.py`` prints supplies ``peak_mem_gb`` (allocator peak + symmetric heaps).
"""

import argparse
import json
import os
import subprocess
import sys

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def run_bench(a, frames: int) -> dict:
    cmd = [sys.executable]
    if a.gpus > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}", "--master-addr", "127.0.0.1",
                "--master-port", str(a.port)]
    cmd += [os.path.join(ROOT, "bench.py"), "--gpus", str(a.gpus), "--frames", str(frames), "--steps", "1", "--warmup", "1",
            "--no-e2e", "--model-type", a.model_type, "--resolution", str(a.resolution[0]), str(a.resolution[1])]
    if a.tp is not None:
        cmd += ["--tp", str(a.tp)]
    if a.cp is not None:
        cmd += ["--cp", str(a.cp)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=a.timeout)
    for line in reversed(r.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    raise RuntimeError(f"bench.py printed no result for {frames} frames:\n{r.stdout[-2000:]}\n{r.stderr[-2000:]}")


def latent_frames(frames: int) -> int:
    return (frames - 1) // 4 + 1


def propose(f0: int, m0: float, f1: int, m1: float, limit_gb: float) -> int:
    """Largest 4k + 1 frame count with predicted peak <= limit, from two (frames, peak GB) measurements."""
    l0, l1 = latent_frames(f0), latent_frames(f1)
    if l1 == l0:
        raise ValueError("the two measurements must differ in latent frames")
    slope = (m1 - m0) / (l1 - l0)                    # GB per latent frame
    if slope <= 0:
        raise ValueError(f"peak memory did not grow with frames ({m0:.1f} -> {m1:.1f} GB)")
    fixed = m0 - slope * l0
    lmax = int((limit_gb - fixed) / slope)
    return max(1, 4 * (lmax - 1) + 1)


def main():
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--tp", type=int, default=None)
    p.add_argument("--cp", type=int, default=None)
    p.add_argument("--model-type", type=str, default="i2v", choices=["t2v", "i2v"])
    p.add_argument("--resolution", type=int, nargs=2, default=[1280, 720])
    p.add_argument("--probe-frames", type=int, nargs=2, default=[33, 65], help="the two small frame counts that are measured")
    p.add_argument("--limit-gb", type=float, default=165.0, help="highest acceptable peak per GPU (of 180 GB)")
    p.add_argument("--no-verify", action="store_true", help="report the proposal without running it")
    p.add_argument("--port", type=int, default=29650)
    p.add_argument("--timeout", type=int, default=1800)
    a = p.parse_args()
    f0, f1 = a.probe_frames
    r0, r1 = run_bench(a, f0), run_bench(a, f1)
    m0, m1 = r0["peak_mem_gb"], r1["peak_mem_gb"]
    best = propose(f0, m0, f1, m1, a.limit_gb)
    out = {"probe": {str(f0): m0, str(f1): m1}, "limit_gb": a.limit_gb, "proposed_frames": best,
           "parallelism": r0["config"]["parallelism"], "n_gpus": a.gpus}
    if not a.no_verify:
        rv = run_bench(a, best)
        out["verified"] = {"frames": best, "peak_mem_gb": rv["peak_mem_gb"], "s_per_step": rv["s_per_step"],
                           "tokens": rv["config"]["seq_len"]}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
