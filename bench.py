"""Benchmark: ring sliding-window attention forward + backward, tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2]

A step is one forward + backward of the public API over one batch of synthetic N(0,1) bf16 inputs.
The default workload is configuration 2 of the benchmark set (B=2, S=32768, 32 q heads / 32 kv heads,
D=128, window 1000).  With --gpus N > 1 (launched under torch.distributed.run, one rank per GPU) the
sequence is sharded over the ranks: by default each rank keeps the 1-GPU chunk (S_global = 32768*N,
"scaling": "weak"); `--scaling strong` keeps S_global = 32768 and splits it.  The other reading is
measured in the same run, untimed for `value`, and reported beside it: "strong" (S_global = 32768 split
over the ranks, with rank 0 alone as the one-GPU figure its efficiency refers to) and "weak_small"
(4096 tokens per rank).

One JSON line is printed by rank 0.  `value` is timed with inputs resident in HBM; `e2e` adds the
host->device copy of q, k, v, dO from pinned memory and the device->host copy of out, dq, dk, dv every
step (three streams: one step's copies overlap the neighbouring steps' compute, none is skipped); `roofline` is the dK/dV backward kernel (the longest one) timed with CUDA events on its stream, `roofline_dq`
and `roofline_fwd` the other two tensor-core kernels;
`roofline_merge` / `roofline_delta` the two streaming kernels against the measured copy bandwidth;
`parity_check` runs four small fixed problems (one-pass halo, window longer than a chunk, sink, packed)
through the public API on the live process group after the timed region and compares every rank's
out, dq, dk, dv with a dense fp32 torch computation of the global problem;
`cpu_baseline` is the dense torch CPU restatement of the reference's test oracle on a bounded slice.

`reference_gpu`, when baseline/_ref holds the reference package, is the reference's own GPU path
(flash-attn 2 + Triton merge) timed on the same GPU and workload in a process of its own
(`--impl reference_gpu` runs just that).
`--impl reference` times that CPU restatement alone (the reference's own attention arithmetic lives in
flash-attn CUDA kernels and has no CPU path; its naive torch oracle is what runs on host cores).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "ring-sliding-window-attention_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

D = 128
WORKLOADS = {
    # name: fn, batch, S (1-GPU tokens per batch row), Hq, Hkv, window, n_sink, seed
    "cfg2": dict(fn="ring_sliding_window_attn", B=2, S=32768, Hq=32, Hkv=32, W=1000, n_sink=0, seed=1),
    "cfg3": dict(fn="ring_sliding_window_attn_varlen", B=1, S=65536, Hq=32, Hkv=8, W=4096, n_sink=0, seed=2),
    "cfg4": dict(fn="ring_streaming_llm_attn", B=1, S=131072, Hq=32, Hkv=8, W=8192, n_sink=1, seed=3),
    "cfg5": dict(fn="ring_sliding_window_attn", B=1, S=262144, Hq=64, Hkv=8, W=65536, n_sink=0, seed=4),
    # reduced case for profiler captures: same kernels, inputs still larger than L2, < 1 GB on the device
    "small": dict(fn="ring_sliding_window_attn", B=1, S=16384, Hq=16, Hkv=16, W=1000, n_sink=0, seed=1),
}
# DRAM bytes (read + write) of one dK/dV-kernel launch on cfg2, from an ncu capture of the "small"
# workload scaled by the number of key tiles; None until measured
TRAFFIC_DKDV_CFG2 = 3.02e9
# cpu sample: a slice of the workload small enough for dense S x S attention on host cores
CPU_SAMPLE = dict(S=4096, H=2)


def cfg3_lengths(total: int):
    """Lengths uniform in [256, 16384] from seed 2, last one truncated to hit `total` exactly."""
    g = torch.Generator().manual_seed(2)
    lens, acc = [], 0
    while acc < total:
        L = int(torch.randint(256, 16385, (1,), generator=g))
        L = min(L, total - acc)
        lens.append(L)
        acc += L
    return lens


def visible_pairs(a: int, b: int, W: int, n_sink: int, seq_starts=None) -> int:
    """Visible (query, key) pairs for queries at global positions [a, b) of one sequence starting at 0."""
    total = 0
    # closed form per piece: query p sees min(p, W) + 1 keys, plus sinks out of the window's reach
    lo = min(b, max(a, W))
    if lo > a:  # p in [a, lo): p + 1 keys
        total += (a + 1 + lo) * (lo - a) // 2
    if b > lo:
        total += (b - lo) * (W + 1)
    if n_sink:
        first = max(a, W + 1)          # p - W > 0: sink 0 out of reach
        for s in range(n_sink):
            f = max(a, W + 1 + s)
            if b > f:
                total += b - f
    return total


def packed_pairs(seq_lens, W: int, n_sink: int) -> int:
    """Visible (query, key) pairs of packed sequences, each starting at its own position 0."""
    return sum(visible_pairs(0, L, W, n_sink) for L in seq_lens)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region, every 20 ms: the figures reported are
    those of the samples taken while the device-resident region ran (`mark()` at its start and end), i.e.
    under load -- a board that idles at its maximum clock drops by a fifth within a few hundred
    milliseconds of these kernels (power cap)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, n_gpus):
        self.n = n_gpus
        self.rows = []
        self.proc = None
        self.marks = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), line.strip()))

    def mark(self):
        self.marks.append(time.monotonic())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, smax, reasons, power = [], [], set(), []
        rows = self.rows
        if len(self.marks) >= 2:  # the samples under load, if there are any (a short region may see none)
            inside = [r for r in rows if self.marks[0] <= r[0] <= self.marks[1] + 0.02]
            rows = inside or rows
        for _t, r in rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 8 or not f[0].isdigit() or int(f[0]) >= self.n:
                continue
            try:
                sm.append(float(f[1])), smax.append(float(f[2])), power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons),
                "sampled": "during the device-resident timed region" if len(self.marks) >= 2 and rows is not self.rows else "whole run"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured", float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))
    return 1590.0, 6650.0, "fallback", 1400.0


def cpu_pass(sample, W, n_sink, seed):
    """One dense fwd+bwd of the oracle on the CPU slice; returns seconds."""
    from oracle.dense_attn import dense_attn_fwd_bwd
    g = torch.Generator().manual_seed(seed)
    S, H = sample["S"], sample["H"]
    q, k, v, do = (torch.randn(1, S, H, D, generator=g).bfloat16().float() for _ in range(4))
    t0 = time.perf_counter()
    dense_attn_fwd_bwd(q, k, v, do, W, None, n_sink)
    return time.perf_counter() - t0


def cpu_tokens_per_s(seconds, sample, wl):
    # the slice covers S tokens of H of the workload's Hq heads: scale to whole-token throughput
    return sample["S"] * (sample["H"] / wl["Hq"]) / seconds


def cpu_small_config():
    """The smallest configuration of the benchmark set (fp32, 1 x 1024 tokens, 4/4 heads of 64, window 128,
    scale 1/8, seed 0) is the one the reference's own CPU-runnable code path covers: its dense torch
    formulation (test/test_local_swa.py:7-95, restated in oracle/), forward + backward, after 2 warm-up
    calls, median of 10.  It executes dense S^2 work; the in-window figure counts 14*D*Hq*pairs."""
    from oracle.dense_attn import dense_attn_fwd_bwd
    S, H, d, W = 1024, 4, 64, 128
    g = torch.Generator().manual_seed(0)
    q, k, v, do = (torch.randn(1, S, H, d, generator=g) for _ in range(4))
    ts = []
    for i in range(12):
        t0 = time.perf_counter()
        dense_attn_fwd_bwd(q, k, v, do, W, 0.125, 0)
        ts.append(time.perf_counter() - t0)
    sec = statistics.median(ts[2:])
    pairs = W * (W + 1) // 2 + (S - W) * (W + 1)
    return {"workload": f"fp32 B=1 S={S} Hq=Hkv={H} D={d} window={W} fwd+bwd, dense torch on the host",
            "ms": 1e3 * sec, "tokens_per_s": S / sec, "in_window_gflops": 14 * d * H * pairs / sec / 1e9,
            "executed_dense_gflops": 14 * d * H * (S * S) / sec / 1e9,
            "threads": torch.get_num_threads(), "cpu_count": os.cpu_count()}


def use_host_cores():
    """torch.distributed.run starts its workers with OMP_NUM_THREADS=1; the CPU arm is meant to use
    the host's cores, so give torch as many threads as a plain start takes (one per physical core)."""
    try:
        n_aff = len(os.sched_getaffinity(0))
    except AttributeError:
        n_aff = os.cpu_count() or 1
    want = max(1, n_aff // 2)
    if torch.get_num_threads() < want:
        torch.set_num_threads(want)


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    use_host_cores()
    for _ in range(args.warmup):
        cpu_pass(CPU_SAMPLE, wl["W"], wl["n_sink"], wl["seed"])
    times = [cpu_pass(CPU_SAMPLE, wl["W"], wl["n_sink"], wl["seed"]) for _ in range(args.steps)]
    total = sum(times)
    val = cpu_tokens_per_s(total / len(times), CPU_SAMPLE, wl)
    sample = (f"dense torch fp32 fwd+bwd of a 1 x {CPU_SAMPLE['S']} x {CPU_SAMPLE['H']}-head slice per step "
              f"(of {wl['Hq']} heads), tokens scaled by the head fraction")
    line = {
        "impl": "reference", "metric": "ring SWA fwd+bwd tokens/s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, wl, args.gpus),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "cpu_small_config": cpu_small_config(),
    }
    print(json.dumps(line), flush=True)


def run_reference_gpu(args, wl):
    """The reference's own GPU path (its ring_swa package from baseline/_ref, flash-attn 2 underneath) on
    one GPU, same workload and timing as the main arm, in a process of its own (the two packages share
    their name).  Prints one JSON line; `unavailable` if the package or its kernels do not run here."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    line = {"impl": "reference_gpu", "metric": "ring SWA fwd+bwd tokens/s", "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "dtype": "bf16", "data": "synthetic"}
    try:
        if not os.path.isdir(os.path.join(ref_dir, "ring_swa")):
            raise RuntimeError("baseline/_ref holds no ring_swa package (install the reference there first)")
        for p_ in (PKG, ROOT):
            while p_ in sys.path:
                sys.path.remove(p_)
        sys.path.insert(0, ref_dir)
        import ring_swa as ref                                # noqa: E402  (the reference's package)
        if not os.path.abspath(ref.__file__).startswith(os.path.abspath(ref_dir)):
            raise RuntimeError("ring_swa did not resolve to baseline/_ref")
        if "varlen" in wl["fn"]:
            raise RuntimeError("only the batch-row workloads are timed on the reference")
        dev = torch.device("cuda", 0)
        B, S, Hq, Hkv, W = wl["B"], wl["S"], wl["Hq"], wl["Hkv"], wl["W"]
        g = torch.Generator(device=dev).manual_seed(wl["seed"] * 1000)
        q, k, v, do = (torch.randn(B, S, h, D, device=dev, generator=g).bfloat16() for h in (Hq, Hkv, Hkv, Hq))
        fn = getattr(ref, wl["fn"])

        def one():
            q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
            fn(q, k, v, W, cp_group=None).backward(do)
            q.grad = k.grad = v.grad = None

        for _ in range(max(args.warmup, 3)):
            one()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        line.update(value=B * S / (ms * 1e-3), ms_per_step=ms,
                    config={"workload": f"{args.workload}: reference {wl['fn']}(cp_group=None) B={B} S={S} Hq={Hq} Hkv={Hkv} "
                                        f"D={D} window={W} fwd+bwd on one GPU through flash-attn"})
    except Exception as e:                                  # noqa: BLE001  (whatever stops it is the answer)
        line["unavailable"] = f"{type(e).__name__}: {str(e)[:300]}"
    print(json.dumps(line), flush=True)


def workload_config(args, wl, n):
    s_rank = wl["S"] if args.scaling == "weak" else wl["S"] // n
    return {"workload": f"{args.workload}: {wl['fn']} B={wl['B']} S_global={s_rank * n} S_per_gpu={s_rank} "
                        f"Hq={wl['Hq']} Hkv={wl['Hkv']} D={D} window={wl['W']} n_sink={wl['n_sink']} fwd+bwd",
            "seed": wl["seed"], "cp_size": n, "l2": "inputs larger than L2 (no flush needed)"}



def dense_reference(q, k, v, do, W, n_sink, cu, scale):
    """Dense fp32 torch attention of the GLOBAL problem on the current device (a checker for small
    problems): q [B,T,Hq,D], k/v [B,T,Hkv,D]; a query at p sees key t of its own sequence with t <= p and
    (p - t <= W or t among the sequence's first n_sink tokens).  Returns out, dq, dk, dv."""
    B, T, Hq, _ = q.shape
    g = Hq // k.shape[2]
    qf, kf, vf = (x.detach().float().requires_grad_(True) for x in (q, k, v))
    pos = torch.arange(T, device=q.device)
    start = torch.zeros(T, dtype=torch.long, device=q.device)
    if cu is not None:
        for a, b in zip(cu[:-1], cu[1:]):
            start[a:b] = a
    same = start[:, None] == start[None, :]
    mask = same & (pos[None, :] <= pos[:, None]) & ((pos[:, None] - pos[None, :] <= W) |
                                                    (pos[None, :] < start[:, None] + n_sink))
    s = torch.einsum("bihd,bjhd->bhij", qf, kf.repeat_interleave(g, 2)) * scale
    s = s.masked_fill(~mask[None, None], float("-inf"))
    o = torch.einsum("bhij,bjhd->bihd", torch.softmax(s, -1), vf.repeat_interleave(g, 2))
    o.backward(do.float())
    return o.detach(), qf.grad, kf.grad, vf.grad


def parity_check(ring_swa, dev, group, n, rank):
    """Four small fixed problems through the public API on the live process group, each rank's slice of
    out, dq, dk, dv against the dense fp32 computation of the global problem (every rank computes that
    itself from the same seed).  Returns the worst errors over cases, tensors and ranks."""
    S = 1024
    T = S * n
    cases = [
        dict(fn="ring_sliding_window_attn", W=300, n_sink=0, cu=None, B=2),      # halo from the previous rank only
        dict(fn="ring_sliding_window_attn", W=2500, n_sink=0, cu=None, B=1),     # window longer than a chunk: several hops, merged
        dict(fn="ring_streaming_llm_attn", W=200, n_sink=1, cu=None, B=1),       # sink fetched from rank 0
        dict(fn="ring_sliding_window_attn_varlen", W=700, n_sink=0, B=1,
             cu=[0, 300, 301, T // 2 + 77, T - 200, T]),                         # packed, sequences crossing rank edges
    ]
    worst_abs, worst_rel, ok = 0.0, 0.0, True
    for ci, c in enumerate(cases):
        gen = torch.Generator(device=dev).manual_seed(4242 + ci)           # the same global tensors on every rank
        Hq, Hkv = 4, 2
        qg, kg, vg, dg = (torch.randn(c["B"], T, h, D, device=dev, generator=gen).bfloat16() for h in (Hq, Hkv, Hkv, Hq))
        scale = D ** -0.5
        ref = dense_reference(qg, kg, vg, dg, c["W"], c["n_sink"], c["cu"], scale)
        sl = slice(rank * S, (rank + 1) * S)
        varlen = c["cu"] is not None
        loc = [x[:, sl].contiguous() for x in (qg, kg, vg, dg)]
        if varlen:
            loc = [x[0] for x in loc]
        ql, kl, vl = (x.detach().requires_grad_(True) for x in loc[:3])
        kw = dict(window_size=c["W"])
        if n > 1:
            kw.update(cp_group=group, cp_size=n, cp_local_rank=rank)
        if varlen:
            kw.update(cu_seqlens=torch.tensor(c["cu"], dtype=torch.int32, device=dev), cp_size=n)
        out = getattr(ring_swa, c["fn"])(ql, kl, vl, **kw)
        out.backward(loc[3])
        for got, want in zip((out.detach(), ql.grad, kl.grad, vl.grad), ref):
            w = want[:, sl] if not varlen else want[0, sl]
            err = (got.float() - w).abs()
            worst_abs = max(worst_abs, float(err.max()))
            worst_rel = max(worst_rel, float((got.float() - w).norm() / w.norm().clamp_min(1e-20)))
            ok = ok and bool((err <= 2e-2 + 1e-2 * w.abs()).all()) and bool(torch.isfinite(got).all())
    t = torch.tensor([worst_abs, worst_rel, 0.0 if ok else 1.0], device=dev, dtype=torch.float64)
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"max_abs_err": t[0].item(), "rel_l2": t[1].item(), "ok": t[2].item() == 0.0 and t[1].item() <= 1e-2,
            "cases": len(cases), "tokens_per_rank": S, "tolerance": "abs <= 2e-2 + 1e-2*|ref|, rel L2 <= 1e-2"}


def time_streaming_kernels(K, q, do, steps):
    """CUDA-event times (ms per launch) of the merge kernel and of the delta kernel on tensors of the
    workload's output shape, and their algorithmic bytes."""
    dev = q.device
    B, S, H, _ = q.shape
    o_a, o_b = q.clone(), do.clone()
    lse_a = torch.randn(B, H, S, device=dev)
    lse_b = torch.randn(B, H, S, device=dev)
    o_c, lse_c = torch.empty_like(o_a), torch.empty_like(lse_a)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for _ in range(3):
        K.merge(o_a, lse_a, o_b, lse_b, out=o_c, lse_out=lse_c)
    ev[0].record()
    for _ in range(steps):
        K.merge(o_a, lse_a, o_b, lse_b, out=o_c, lse_out=lse_c)
    ev[1].record()
    torch.cuda.synchronize()
    merge_ms = ev[0].elapsed_time(ev[1]) / steps
    merge_bytes = B * S * H * (3 * D * 2 + 3 * 4)
    # the delta kernel alone: an INIT call without K/V gradient buffers launches nothing else
    from ring_swa import _C
    ws = K.bwd_workspace(q)
    kv = q[:, :, :1]
    span = [K.KVSpan(kv, kv, 0)]
    for _ in range(3):
        K.bwd(q, span, o_a, lse_a, do, o_c, 1, 0, 1.0, workspace=ws, flags=_C.BWD_INIT)
    ev[0].record()
    for _ in range(steps):
        K.bwd(q, span, o_a, lse_a, do, o_c, 1, 0, 1.0, workspace=ws, flags=_C.BWD_INIT)
    ev[1].record()
    torch.cuda.synchronize()
    delta_ms = ev[0].elapsed_time(ev[1]) / steps
    delta_bytes = B * S * H * (2 * D * 2 + 4 + 2 * 4)      # out and dO read once, lse read, two float rows written
    return merge_ms, merge_bytes, delta_ms, delta_bytes


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_gpu"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the strong / weak_small series")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip timing the reference's GPU path (baseline/_ref)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    wl = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference(args, wl)
        return
    if args.impl == "reference_gpu":
        run_reference_gpu(args, wl)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torch.distributed.run with --nproc-per-node {args.gpus}")
    n = world
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    group = None
    if n > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD

    import ring_swa
    from ring_swa import _C
    from ring_swa import _kernels as K

    fn = getattr(ring_swa, wl["fn"])
    varlen = "varlen" in wl["fn"]
    S = wl["S"] if args.scaling == "weak" else wl["S"] // n      # tokens per rank
    S_g = S * n
    B, Hq, Hkv, W, n_sink = wl["B"], wl["Hq"], wl["Hkv"], wl["W"], wl["n_sink"]
    lead = (S,) if varlen else (B, S)
    g = torch.Generator(device=dev).manual_seed(wl["seed"] * 1000 + rank)
    q, k, v, do = (torch.randn(*lead, h, D, device=dev, generator=g).bfloat16() for h in (Hq, Hkv, Hkv, Hq))
    kw = dict(window_size=W)
    if n > 1:
        kw.update(cp_group=group, cp_size=n, cp_local_rank=rank)
    seq_lens = [S_g] * B
    if varlen:
        seq_lens = cfg3_lengths(S_g)
        cu = [0]
        for L in seq_lens:
            cu.append(cu[-1] + L)
        kw.update(cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=dev), cp_size=n)
    if n_sink and n_sink != 1:
        kw["num_sink_tokens"] = n_sink

    def step(qq, kk, vv, dd):
        qq.requires_grad_(True), kk.requires_grad_(True), vv.requires_grad_(True)
        out = fn(qq, kk, vv, **kw)
        out.backward(dd)
        grads = (qq.grad, kk.grad, vv.grad)
        qq.grad = kk.grad = vv.grad = None
        return out.detach(), grads

    def sync_all():
        torch.cuda.synchronize()
        if n > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # The first steps of a multi-rank job also set up NCCL's peer-to-peer channels (seen once as a
    # 5 ms outlier inside the timed region right after a box came up): a few extra untimed steps.
    for _ in range(args.warmup + (4 if n > 1 else 0)):
        step(q, k, v, do)
    sync_all()
    K.check_device_status(dev)

    # ---------------------------------------------------------------- device-resident timing
    sampler = ClockSampler(n) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    K.fwd_events, K.bwd_main_events = [], []
    launches0 = K.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    if sampler:
        sampler.mark()
    e0.record()
    for _ in range(args.steps):
        step(q, k, v, do)
    e1.record()
    sync_all()
    if sampler:
        sampler.mark()
    ms = e0.elapsed_time(e1)
    launches = K.launch_count - launches0
    lib = _C.lib()
    fwd_ms = sum(lib.rswa_event_elapsed_ms(a, b) for a, b in K.fwd_events) / args.steps
    bwd_ms = sum(lib.rswa_event_elapsed_ms(a, m) for a, m, b in K.bwd_main_events) / args.steps     # dK/dV kernel
    dq_ms = sum(lib.rswa_event_elapsed_ms(m, b) for a, m, b in K.bwd_main_events) / args.steps      # dQ kernel
    for evs in K.fwd_events + K.bwd_main_events:
        for e in evs:
            lib.rswa_event_destroy(e)
    K.fwd_events = K.bwd_main_events = None
    K.check_device_status(dev)

    # ---------------------------------------------------------------- end to end (host buffers)
    e2e = None
    if not args.no_e2e:
        host_in = [x.detach().cpu().pin_memory() for x in (q, k, v, do)]
        host_out = [torch.empty_like(x, device="cpu").pin_memory() for x in (q, q, k, v)]
        dev_in = [torch.empty_like(x) for x in (q, k, v, do)]
        h2d = sum(x.numel() * x.element_size() for x in host_in)
        d2h = sum(x.numel() * x.element_size() for x in host_out)

        # Three streams, two sets of device input buffers: step i's host->device copies run while
        # step i-1 computes and step i-2's results go back to the host, as an input pipeline that
        # double-buffers would do it.  Every step still copies all of its inputs in and all of its
        # results (out, dq, dk, dv) out inside the timed region.
        main = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        dev_in2 = [dev_in, [torch.empty_like(x) for x in (q, k, v, do)]]
        free_ev = [None, None]      # inputs of a set may be overwritten once the step that read them is done
        out_ev = [None]             # the host result buffers are reused by every step

        def e2e_step(i):
            cur = dev_in2[i & 1]
            with torch.cuda.stream(s_in):
                if free_ev[i & 1] is not None:
                    s_in.wait_event(free_ev[i & 1])
                for d_, h_ in zip(cur, host_in):
                    d_.copy_(h_, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            main.wait_event(ready)
            out, grads = step(cur[0].detach(), cur[1].detach(), cur[2].detach(), cur[3])
            done = torch.cuda.Event()
            done.record(main)
            free_ev[i & 1] = done
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for h_, d_ in zip(host_out, (out,) + grads):
                    d_.record_stream(s_out)
                    h_.copy_(d_, non_blocking=True)

        for i in range(2):
            e2e_step(i)
        sync_all()
        n_e2e = max(4, min(args.steps, 10))
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(main)
        for i in range(n_e2e):
            e2e_step(i)
        main.wait_stream(s_out)     # the last results are on the host when the clock stops
        f1.record(main)
        sync_all()
        e2e_ms = f0.elapsed_time(f1) / n_e2e
    clocks = sampler.stop() if sampler else None

    # ---------------------------------------------------------------- the other scaling readings (untimed for `value`)
    def timed_series(S_rank, ranks, kw_run):
        """ms per step (this rank) of `steps` steps at S_rank tokens per rank, after `warmup` steps."""
        gg = torch.Generator(device=dev).manual_seed(wl["seed"] * 1000 + 77 + rank)
        qq, kk, vv, dd = (torch.randn(B, S_rank, h, D, device=dev, generator=gg).bfloat16() for h in (Hq, Hkv, Hkv, Hq))

        def one():
            qq.requires_grad_(True), kk.requires_grad_(True), vv.requires_grad_(True)
            fn(qq, kk, vv, **kw_run).backward(dd)
            qq.grad = kk.grad = vv.grad = None

        for _ in range(args.warmup):
            one()
        if ranks > 1:
            sync_all()
        else:
            torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(args.steps):
            one()
        a1.record()
        torch.cuda.synchronize()
        t_ms = a0.elapsed_time(a1) / args.steps
        if ranks > 1:      # where the compute stream's time goes, phase by phase (5 more steps, untimed)
            phase_tables.append(measure_phases(one))
        return t_ms

    from ring_swa import _ring as ring_impl
    phase_tables = []

    def measure_phases(one_step, k_steps=5):
        """[ms per step of each phase of ring_swa._ring.PHASES] on this rank's compute stream."""
        sync_all()
        ring_impl.phase_timing(True)
        for _ in range(k_steps):
            one_step()
        t = ring_impl.phase_times()
        ring_impl.phase_timing(False)
        return [t[name] / k_steps for name in ring_impl.PHASES]

    if n > 1 and not args.no_extra:
        phase_tables.append(measure_phases(lambda: step(q, k, v, do)))

    extra_ms = [0.0, 0.0, 0.0]      # strong at n ranks, rank 0 alone on the whole sequence, weak_small
    do_extra = not varlen and not args.no_extra and args.scaling == "weak"
    S_small = 4096
    if do_extra:
        if n > 1:
            extra_ms[0] = timed_series(wl["S"] // n, n, kw)
            sync_all()
            if rank == 0:       # the one-GPU time of the same global sequence, the other ranks idle
                extra_ms[1] = timed_series(wl["S"], 1, dict(window_size=W))
            sync_all()
        extra_ms[2] = timed_series(S_small, n, kw)
        sync_all()

    # ---------------------------------------------------------------- streaming kernels, parity
    stream_k = time_streaming_kernels(K, q if not varlen else q[None], do if not varlen else do[None], 10) if rank == 0 else None
    sync_all()
    parity = parity_check(ring_swa, dev, group, n, rank)
    sync_all()
    K.check_device_status(dev)

    # ---------------------------------------------------------------- reduce over ranks
    stats = torch.tensor([ms, fwd_ms, bwd_ms, e2e_ms if not args.no_e2e else 0.0, dq_ms] + extra_ms, device=dev,
                         dtype=torch.float64)
    if n > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms, fwd_ms, bwd_ms, e2e_ms, dq_ms, strong_ms, alone_ms, small_ms = stats.tolist()
    phases = None
    if phase_tables:       # rows: the main (weak) run, then strong and weak_small where they ran; max over ranks
        pt = torch.tensor(phase_tables, device=dev, dtype=torch.float64)
        dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        phases = [{name: round(v_, 4) for name, v_ in zip(ring_impl.PHASES, row) if v_ > 0} for row in pt.tolist()]

    if rank == 0:
        tokens = B * S_g
        ms_step = ms / args.steps
        peak_tf, peak_gbs, peak_kind, peak_sustained = measured_peaks()
        peak_name = "bf16_tflops (burst)"
        # Kernels that run for tens of milliseconds pull the board to its power cap and the SM clock
        # drops: for such a run the sustained figure is the denominator, for short kernels at full
        # clock the burst figure.
        if clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and "sw_power_cap" in clocks.get("reasons", []) \
                and clocks["sm_mhz"] < 0.9 * clocks["sm_max_mhz"]:
            peak_tf, peak_name = peak_sustained, "bf16_tflops_sustained (SM clock below 90 % of max under the power cap)"
        if varlen:
            pairs_total = packed_pairs(seq_lens, W, n_sink)
        else:
            pairs_total = B * visible_pairs(0, S_g, W, n_sink)
        # work is near-uniform over ranks except the first ones; the slowest rank is the last
        pairs_rank = B * visible_pairs(S_g - S, S_g, W, n_sink) if not varlen else pairs_total / n
        # algorithmic FLOPs on visible pairs: dK/dV kernel 4 products (S^T, dP^T, dV, dK), dQ kernel 3 (S, dP,
        # dQ; the recomputed S and dP are counted because the kernel executes them), forward 2
        flops_bwd = 8 * D * Hq * pairs_rank
        flops_dq = 6 * D * Hq * pairs_rank
        flops_fwd = 4 * D * Hq * pairs_rank
        ach_bwd = flops_bwd / (bwd_ms * 1e-3) / 1e12
        ach_dq = flops_dq / (dq_ms * 1e-3) / 1e12
        ach_fwd = flops_fwd / (fwd_ms * 1e-3) / 1e12
        line = {
            "metric": "ring SWA fwd+bwd tokens/s", "value": tokens / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(args, wl, n),
            "tflops_per_gpu_in_window": 14 * D * Hq * pairs_total / n / (ms_step * 1e-3) / 1e12,
            "frac_of_bf16_peak": 14 * D * Hq * pairs_total / n / (ms_step * 1e-3) / 1e12 / peak_tf,
            "bf16_peak_used": {"tflops": peak_tf, "which": peak_name,
                               "frac_of_burst_peak": 14 * D * Hq * pairs_total / n / (ms_step * 1e-3) / 1e12 / measured_peaks()[0]},
            "roofline": {"kernel": "rswa_bwd_kernel (dK/dV)", "bound": "tensor", "achieved": ach_bwd, "peak": peak_tf,
                         "unit": "TFLOP/s", "frac": ach_bwd / peak_tf, "traffic": TRAFFIC_DKDV_CFG2 if args.workload == "cfg2" and n == 1 else None,
                         "peak_source": f"{peak_kind} {peak_name}", "ms_per_launch": bwd_ms,
                         "algorithmic_flops_per_launch": flops_bwd},
            "roofline_dq": {"kernel": "rswa_dq_kernel", "bound": "tensor", "achieved": ach_dq, "peak": peak_tf,
                            "unit": "TFLOP/s", "frac": ach_dq / peak_tf, "ms_per_launch": dq_ms,
                            "algorithmic_flops_per_launch": flops_dq},
            "roofline_fwd": {"kernel": "rswa_fwd_kernel", "bound": "tensor", "achieved": ach_fwd, "peak": peak_tf,
                             "unit": "TFLOP/s", "frac": ach_fwd / peak_tf, "ms_per_launch": fwd_ms},
            "gpu_launches": launches,
            "clocks": clocks,
            "parity_check": parity,
        }
        if stream_k is not None:
            merge_ms, merge_bytes, delta_ms, delta_bytes = stream_k
            for name, kern, t_ms, nbytes in (("roofline_merge", "merge_kernel", merge_ms, merge_bytes),
                                            ("roofline_delta", "delta_kernel", delta_ms, delta_bytes)):
                gbs = nbytes / (t_ms * 1e-3) / 1e9
                line[name] = {"kernel": kern, "bound": "hbm", "achieved": gbs, "peak": peak_gbs, "unit": "GB/s",
                              "frac": gbs / peak_gbs, "ms_per_launch": t_ms, "algorithmic_bytes_per_launch": nbytes,
                              "peak_source": f"{peak_kind} hbm_gbs (copy)"}
        if do_extra:
            def scaling_obj(S_glob, t_ms, n_ranks):
                pr = B * visible_pairs(0, S_glob, W, n_sink)
                return {"S_global": S_glob, "S_per_gpu": S_glob // n_ranks, "ms_per_step": t_ms,
                        "tokens_per_s": B * S_glob / (t_ms * 1e-3),
                        "tflops_per_gpu": 14 * D * Hq * pr / n_ranks / (t_ms * 1e-3) / 1e12}
            if n > 1:
                line["strong"] = scaling_obj(wl["S"], strong_ms, n)
                line["strong"]["one_gpu_ms_per_step"] = alone_ms
                line["strong"]["efficiency_vs_n1"] = alone_ms / (n * strong_ms)
            else:
                line["strong"] = scaling_obj(wl["S"], ms_step, 1)
                line["strong"]["efficiency_vs_n1"] = 1.0
            line["weak_small"] = scaling_obj(S_small * n, small_ms, n)
        if phases:
            # ms per step of each host-visible phase on the compute stream, max over ranks (CUDA events):
            # the *_wait entries are the time the compute stream stood still waiting for halo data
            line["phases_ms"] = phases[0]
            if do_extra and len(phases) >= 3:
                line["strong"]["phases_ms"] = phases[1]
                line["weak_small"]["phases_ms"] = phases[2]
        if not args.no_e2e:
            line["e2e"] = {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d * n,
                           "d2h_bytes_per_step": d2h * n, "ms_per_step": e2e_ms}
        if n == 1 and not args.no_ref_gpu and os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "ring_swa")):
            # the reference's GPU path on the same GPU right after ours, for the record (not the reference arm)
            try:
                r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference_gpu", "--workload",
                                    args.workload, "--steps", str(min(args.steps, 10)), "--warmup", "3"],
                                   capture_output=True, text=True, timeout=300)
                ref_line = json.loads(r.stdout.strip().splitlines()[-1])
            except Exception as e:                          # noqa: BLE001
                ref_line = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
            line["reference_gpu"] = {k_: ref_line.get(k_) for k_ in ("value", "unit", "ms_per_step", "unavailable", "config")
                                     if ref_line.get(k_) is not None}
            if ref_line.get("ms_per_step"):
                line["reference_gpu"]["speedup_of_this_build"] = ref_line["ms_per_step"] / ms_step
        if n == 1 and not args.no_cpu_baseline:
            use_host_cores()
            t = [cpu_pass(CPU_SAMPLE, W, n_sink, wl["seed"])]          # first call warms torch up
            t0 = time.perf_counter()
            runs = []
            while time.perf_counter() - t0 < 10.0 or len(runs) < 2:
                runs.append(cpu_pass(CPU_SAMPLE, W, n_sink, wl["seed"]))
            line["cpu_baseline"] = {
                "value": cpu_tokens_per_s(statistics.median(runs), CPU_SAMPLE, wl), "unit": "tokens/s",
                "cores": torch.get_num_threads(), "kind": "port",
                "sample": f"{len(runs)} dense fp32 fwd+bwd passes over a 1 x {CPU_SAMPLE['S']} x {CPU_SAMPLE['H']}-head "
                          f"slice (of {Hq} heads), median; tokens scaled by the head fraction"}
            try:
                line["cpu_small_config"] = cpu_small_config()
            except Exception as e:                          # noqa: BLE001  (an extra figure must not cost the line)
                line["cpu_small_config"] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
        print(json.dumps(line), flush=True)
    if n > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
