"""Benchmark of the slot-scan hot path: forward + backward of the hard-address scan at the sh25 training shape.

    python bench.py [--gpus N] [--steps K] [--warmup W]            this build's CUDA path
    python bench.py --impl reference [...]                          the CPU implementation timed on the host cores
    torchrun ... bench.py --gpus N ...                              one rank per GPU, the batch sharded over the ranks

One step = one forward + backward pass of the scan over one batch of T=1024-token sequences x 6 heads (N=192 slots,
dk=dv=128, snapshot stride 8, bf16 token streams and snapshots, float32 state and accumulation), on seeded synthetic
inputs with the benchmark's distributions.  The global batch is 64 sequences at every GPU count (strong scaling:
64 / N sequences per rank, no data-path collective); `--scaling weak` keeps 64 sequences per GPU instead.
Prints ONE JSON line:
  value      tokens/s, whole job, inputs resident in HBM, device-timed (CUDA events, max over ranks)
  e2e        the same through the public Python API with HOST (pinned) inputs: H2D of k,q,v,gate,fr and D2H of every
             input gradient inside the timed region
  roofline   the dominant kernel's algorithmic bytes / its event-timed duration against the measured HBM peak;
             .step the same for the whole step, .touched_* with the bytes the kernels are obliged to move on THESE
             inputs (snapshot-gradient rows of slots that never were candidates reach no input and are skipped),
             .fill the step on inputs that use every slot
  extra      one GPU only: the reference's own CUDA scan timed on this GPU (when staged under baseline/_ref/), the
             writer epilogue and one reader layer's cosine read over the snapshots of the same scan
  cpu_baseline  the CPU oracle (C, OpenMP) on a bounded sample of the same workload, on this box's host cores
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "smal-memory-llm_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

METRIC = "slot-scan tokens/s per B200 (fwd+bwd, sh25 shape), % HBM roofline, 1/2/4/8 GPU"
SHAPE = dict(B=64, T=1024, H=6, N=192, DK=128, DV=128, G=8)
FALLBACK_HBM_GBS = 6650.0


_OUT = None


def claim_stdout():
    """Keep the process's real stdout for the one JSON line and point file descriptor 1 at stderr for everything else:
    libraries print there too (NCCL writes its version banner to stdout from C code)."""
    global _OUT
    if _OUT is None:
        sys.stdout.flush()
        _OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line):
    out = _OUT if _OUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def algorithmic_bytes_per_token_head(N, DK, DV, G, e_in, e_s):
    """Drop-in form, per token and head: forward reads k,q,v + gate,fr and writes the snapshots; backward re-reads the
    inputs, reads the snapshot gradients and writes dk,dq,dv,dgate,dfr.  Logs and scratch are not counted."""
    tok = (2 * DK + DV) * e_in + 8
    snap = N * (DK + DV) * e_s / G
    return dict(fwd=tok + snap, bwd=tok + snap + tok, total=3 * tok + 2 * snap, tok=tok, snap=snap)


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE, text=True)
            self.thr = threading.Thread(target=self._read, daemon=True)
            self.thr.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def max_over_ranks(values, device):
    """Element-wise MAX of a list of floats over all ranks (the time of a multi-GPU step is its slowest rank's)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def whole_job_tokens_per_s(B_per_rank, T, world, steps, ms):
    """Every rank scans its own B_per_rank sequences; the job's throughput counts all of them."""
    return B_per_rank * T * world * steps / (ms * 1e-3)


def shard_of_batch(global_B, world, rank, scaling):
    """(first sequence, number of sequences) of this rank.  strong: the global batch is split evenly (the remainder
    goes to the first ranks); weak: every rank holds `global_B` sequences of its own."""
    if scaling == "weak" or world == 1:
        return rank * global_B, global_B
    base, rem = divmod(global_B, world)
    n = base + (1 if rank < rem else 0)
    return rank * base + min(rank, rem), n


def make_host_inputs(B, T, H, DK, DV, seed, dist="bench"):
    from tests.scan_cases import make_inputs
    return make_inputs(dist, B, T, H, DK, DV, seed=seed)


# ------------------------------------------------------------------------------------------------------------------
def host_threads():
    """All host cores the process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1 for its children)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_sample_batch(threads, H):
    """Sequences of the CPU sample: the oracle runs one (sequence, head) scan per OpenMP task, so the sample holds at
    least two tasks per core (dynamic schedule) -- every core has work for the whole step."""
    return max(2, math.ceil(2 * threads / H))


def cpu_leg(steps, warmup, threads=None, budget_s=60.0):
    """The CPU implementation of the same path: the C oracle (float32, OpenMP over (sequence, head)), forward + backward,
    on a bounded sample: `sample_B` sequences of the full T / H / N / D, every host core busy."""
    import numpy as np
    from oracle import oracle as O
    threads = threads or host_threads()
    flags = O.use_timed_build()
    O.set_threads(threads)
    s = SHAPE
    sample_B = min(cpu_sample_batch(threads, s["H"]), s["B"])
    inp = make_host_inputs(sample_B, s["T"], s["H"], s["DK"], s["DV"], seed=0)
    kw = dict(N=s["N"], temp=16.0, G=s["G"], hard=True, q=inp["q"], occ_bin=True, dtype=np.float32)
    NB = (s["T"] + s["G"] - 1) // s["G"]
    rng = np.random.default_rng(7)
    wk = rng.standard_normal((sample_B, NB, s["H"], s["N"], s["DK"]), dtype=np.float32)
    wv = rng.standard_normal((sample_B, NB, s["H"], s["N"], s["DV"]), dtype=np.float32)

    def step():
        O.scan_fwd(inp["k"], inp["v"], inp["gate"], inp["fr"], **kw)
        O.scan_bwd(inp["k"], inp["v"], inp["gate"], inp["fr"], dkbuf=wk, dvbuf=wv, detach_addr=True, **kw)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        step()
        done += 1
        if time.perf_counter() - t0 > budget_s:          # keep the whole run within minutes on a slow host
            break
    dt = time.perf_counter() - t0
    toks = sample_B * s["T"] * done
    out = dict(value=toks / dt, ms_per_step=1e3 * dt / done, cores=O.threads(), steps=done, sample_B=sample_B, build=flags,
               sample="%d of %d sequences (%d OpenMP tasks on %d threads), full T=%d H=%d N=%d D=%d G=%d, float32, fwd+bwd"
                      % (sample_B, s["B"], sample_B * s["H"], O.threads(), s["T"], s["H"], s["N"], s["DK"], s["G"]))
    # config 0 as specified: B=2, T=256, forward only, float32 (scan -> epilogue -> read), the whole case, not a sample
    c0 = make_host_inputs(2, 256, s["H"], s["DK"], s["DV"], seed=0)
    rq = np.random.default_rng(1)
    qr = rq.standard_normal((2, 256, s["H"], 1, s["DK"])).astype(np.float32)
    sharp = (np.log1p(np.exp(rq.standard_normal((2, 256, s["H"], 1)))) + 1).astype(np.float32)

    def cfg0():
        r = O.scan_fwd(c0["k"], c0["v"], c0["gate"], c0["fr"], N=s["N"], temp=16.0, G=s["G"], hard=True, q=c0["q"],
                       occ_bin=True, dtype=np.float32)
        ki, va = O.epilogue(r["kbuf"], dtype=np.float32)
        O.read_fwd(qr, sharp, r["kbuf"], r["vbuf"], ki, va, s["G"], dtype=np.float32)

    cfg0()
    t0 = time.perf_counter()
    for _ in range(3):
        cfg0()
    out["config0"] = {"tokens_per_s": 3 * 2 * 256 / (time.perf_counter() - t0), "workload": "config0: B=2 T=256 H=6 N=192 "
                      "D=128 G=8, float32, forward scan + epilogue + read, whole case (12 OpenMP tasks)"}
    return out


def reference_kernel_leg(B, T, H, N, D, G, steps, warmup, dist="bench", seed=0, timeout_s=600):
    """The reference's own CUDA scan (runtime-compiled, float32 streams and snapshots) on this GPU, in a process of its
    own: baseline/time_reference_kernel.py over the modules staged under baseline/_ref/ (git-ignored).  A secondary
    baseline beside the CPU arm; returns {"unavailable": why} when the staging is absent or the run fails."""
    script = os.path.join(ROOT, "baseline", "time_reference_kernel.py")
    if not os.path.isfile(os.path.join(ROOT, "baseline", "_ref", "gqa25", "slotkern_cuda.py")):
        return {"unavailable": "baseline/_ref/gqa25 is not staged (baseline/stage_reference.py needs a reference checkout)"}
    cmd = [sys.executable, script] + [str(x) for x in (B, T, H, N, D, G, steps, warmup, dist, seed)]
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s)
        for ln in reversed(out.stdout.strip().splitlines()):
            if ln.startswith("{"):
                return json.loads(ln)
        return {"unavailable": "rc=%d: %s" % (out.returncode, (out.stderr.strip().splitlines() or ["no output"])[-1][:300])}
    except Exception as e:                                             # noqa: BLE001 -- a baseline must not fail the bench
        return {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:300])}


def run_reference(args, rank, world):
    if rank != 0:
        return
    r = cpu_leg(max(1, args.steps), args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": r["steps"], "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config1: slot-scan fwd+bwd, B=64 T=1024 H=6 N=192 dk=dv=128 G=8 (CPU sample: see cpu_baseline.sample)",
                       "global_batch": SHAPE["B"], "seq_len": SHAPE["T"], "l2": "n/a (host)"},
            "cpu_baseline": {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port", "sample": r["sample"],
                             "build": r["build"], "config0": r["config0"]},
            "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    try:
        import torch
        if torch.cuda.is_available():
            line["reference_gpu_kernel"] = reference_kernel_leg(SHAPE["B"] // max(1, args.gpus), SHAPE["T"], SHAPE["H"], SHAPE["N"],
                                                               SHAPE["DK"], SHAPE["G"], max(3, args.steps), max(3, args.warmup))
    except ImportError:
        pass
    emit(line)


# ------------------------------------------------------------------------------------------------------------------
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures summarised under profiles/
# (each taken at B = 8 sequences; traffic is proportional to the batch, so a launch over B sequences moves B / 8 of it).
# A kernel that changed since its capture is taken out of this table until it is captured again.
NCU_TRAFFIC_B8 = {
    "addr_fwd||zero_fill": (25.6e6 + 493.8e6, "profiles/addr_fwd_128_bf16_small_case.md + profiles/zero_rows_bulk_128_bf16_small_case.md"),
    "replay_rows_k": (25.6e6 + 52.3e6, "profiles/replay_rows_128_bf16_small_case.md"),
    "rows_bwd_k": (107.8e6 + 15.7e6, "profiles/rows_bwd_128_bf16_small_case.md"),
    "addr_bwd": (52.43e6 + 1.18e6, "profiles/addr_bwd_gather_128_bf16_small_case.md"),
}


class ScanJob:
    """One rank's share of the workload: inputs on the host (pinned) and on the device, upstream gradients, the step."""

    def __init__(self, S, dev, B, T, H, N, DK, DV, G, seed, dist):
        import torch
        self.S, self.dev, self.dims = S, dev, (B, T, H, N, DK, DV, G)
        NB = (T + G - 1) // G
        inp = make_host_inputs(B, T, H, DK, DV, seed=seed, dist=dist)
        bf = torch.bfloat16
        self.host = {n: inp[n].to(bf).contiguous().pin_memory() for n in ("k", "q", "v")}
        self.host.update({n: inp[n].float().contiguous().pin_memory() for n in ("gate", "fr")})
        self.devin = {n: t.to(dev) for n, t in self.host.items()}
        self.temp = torch.tensor([16.0], device=dev)
        gen = torch.Generator(device=dev).manual_seed(7 + seed)
        self.dkb = torch.randn(B, NB, H, N, DK, device=dev, dtype=bf, generator=gen)
        self.dvb = torch.randn(B, NB, H, N, DV, device=dev, dtype=bf, generator=gen)

    def scan(self, x, sl=slice(None)):
        import torch
        B, T, H, N, DK, DV, G = self.dims
        k, q, v = (x[n].detach().requires_grad_() for n in ("k", "q", "v"))
        g, fr = x["gate"].detach().requires_grad_(), x["fr"].detach().requires_grad_()
        tp = self.temp.detach().requires_grad_()
        kb, vb = self.S.kv_scan_g(k, v, g, fr, N, tp, G=G, hard=True, hard_gate=False, detach_addr=True, q=q, occ_bin=True,
                                  out_dtype=torch.bfloat16)
        torch.autograd.backward([kb, vb], [self.dkb[sl], self.dvb[sl]])
        return k.grad, q.grad, v.grad, g.grad, fr.grad, tp.grad

    def step(self):
        return self.scan(self.devin)

    def touched_bytes(self):
        """Bytes the kernels are obliged to move on these inputs: as the algorithmic figure, but of the snapshot
        gradients only the rows that can reach an input -- row n from the block in which it first became a candidate
        (tfirst of the forward log).  The forward has to write every snapshot row, zeros included."""
        import torch
        B, T, H, N, DK, DV, G = self.dims
        NB = (T + G - 1) // G
        x = self.devin
        with torch.no_grad():
            lg = self.S.scan_with_log(x["k"], x["v"], x["gate"], x["fr"], N, 16.0, G=G, q=x["q"], occ_bin=True,
                                      out_dtype=torch.bfloat16)
        tf = lg["tfirst"].long()                                         # (B*H, N): first token at which row n is a candidate
        blocks = torch.where(tf < T, NB - tf // G, torch.zeros_like(tf))  # snapshots taken at or after the block that holds tfirst
        rows_read = int(blocks.sum())
        used = float((tf < T).float().sum(1).mean())
        ab = algorithmic_bytes_per_token_head(N, DK, DV, G, 2, 2)
        tok_heads = B * T * H
        full = ab["total"] * tok_heads
        snap_grad_full = ab["snap"] * tok_heads
        snap_grad_touched = rows_read * (DK + DV) * 2
        del lg
        return dict(step=full - snap_grad_full + snap_grad_touched, rows_bwd=snap_grad_touched + 2 * (DK + DV) * 2 * tok_heads,
                    slots_used_mean=used)


def timed(job, steps, barrier, clock_index=None):
    """`steps` calls of job.step() between two events on the current stream, barrier + synchronize on both sides.
    The per-kernel event times come from a few more steps AFTER the timed region: the library's per-launch events
    cost two event creations and two records per kernel on the host, which a step of a millisecond (few sequences per
    GPU) would feel."""
    import torch
    from slotscan_b200 import _lib
    _lib.profile_enable(False)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clk = ClockSampler(clock_index) if clock_index is not None else None
    if clk:
        clk.__enter__()
    barrier()
    e0.record()
    for _ in range(steps):
        job.step()
    e1.record()
    barrier()
    if clk:
        clk.__exit__()
    _lib.profile_enable(True)
    _lib.profile_read()
    psteps = min(steps, 5)
    for _ in range(psteps):
        job.step()
    torch.cuda.synchronize()
    prof = _lib.profile_read()
    _lib.profile_enable(False)
    # counts and times as of the timed region: the same launches per step, `steps` steps
    prof = {n: (c * steps // psteps, t * steps / psteps) for n, (c, t) in prof.items()}
    return e0.elapsed_time(e1), prof, (clk.summary() if clk else None)


def run_gpu(args, rank, local_rank, world):
    import torch
    import slotscan_b200 as S

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: this build has no CPU path for the scan")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist_on = world > 1
    if dist_on:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    s = dict(SHAPE)
    if args.B:
        s["B"] = args.B
    if args.T:
        s["T"] = args.T
    GB, T, H, N, DK, DV, G = (s[n] for n in ("B", "T", "H", "N", "DK", "DV", "G"))
    scaling = args.scaling
    first, B = shard_of_batch(GB, world, rank, scaling)
    global_B = GB * world if scaling == "weak" else GB
    if B < 1:
        raise RuntimeError("fewer sequences than ranks")
    # every rank draws its own sequences (seeded by rank): the scan never looks across sequences
    job = ScanJob(S, dev, B, T, H, N, DK, DV, G, seed=rank, dist=args.dist)

    def barrier():
        if dist_on:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        job.step()
    barrier()
    # ---- device-timed leg: inputs resident in HBM ----
    ms, prof, clocks = timed(job, args.steps, barrier, clock_index=local_rank)

    # ---- end-to-end leg: host inputs in, input gradients out, every step ----
    # The batch goes through in P chunks on P streams, so that the host->device copy of one chunk, the kernels of
    # another and the device->host copy of a third overlap (sequences are independent; the copies use both directions
    # of the link).  All through the public call, kv_scan_g, as a user would write it.
    P = args.e2e_chunks
    while P > 1 and (B % P or B < 2 * P):
        P //= 2
    bs = B // P
    streams = [torch.cuda.Stream(device=dev) for _ in range(P)]
    host = job.host
    # One pinned staging buffer per chunk and direction: [k | q | v | gate | fr] of the chunk's sequences back to back, so
    # that a chunk moves in ONE host->device copy and its gradients (+ dtemp) leave in ONE device->host copy.  The
    # "application" owns these buffers: producing the inputs into them / consuming the gradients from them is its side.
    names = ("k", "q", "v", "gate", "fr")
    sizes = [host[n][:bs].numel() * host[n].element_size() for n in names]
    offs = [sum(sizes[:i]) for i in range(len(names))]
    chunk_bytes = (sum(sizes) + 4 + 255) // 256 * 256             # + dtemp on the way out
    hin = [torch.empty(chunk_bytes, dtype=torch.uint8).pin_memory() for _ in range(P)]
    hout = [torch.empty(chunk_bytes, dtype=torch.uint8).pin_memory() for _ in range(P)]
    din = [torch.empty(chunk_bytes, dtype=torch.uint8, device=dev) for _ in range(P)]
    dout = [torch.empty(chunk_bytes, dtype=torch.uint8, device=dev) for _ in range(P)]

    def view(flat, j):                                            # tensor j of a chunk inside its staging buffer
        t = host[names[j]]
        return flat[offs[j]:offs[j] + sizes[j]].view(t.dtype).view((bs,) + tuple(t.shape[1:]))
    for i in range(P):                                            # the inputs, as the application would have left them
        for j, n in enumerate(names):
            view(hin[i], j).copy_(host[n][i * bs:(i + 1) * bs])

    def e2e_step():
        cur = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(cur)
        for i, st in enumerate(streams):
            sl = slice(i * bs, (i + 1) * bs)
            st.wait_event(start)
            with torch.cuda.stream(st):
                din[i].copy_(hin[i], non_blocking=True)
                x = {n: view(din[i], j) for j, n in enumerate(names)}
                grads = job.scan(x, sl)
                for j in range(5):
                    view(dout[i], j).copy_(grads[j])
                dout[i][offs[4] + sizes[4]:offs[4] + sizes[4] + 4].view(torch.float32).copy_(grads[5].reshape(1))
                hout[i].copy_(dout[i], non_blocking=True)
        for st in streams:
            cur.wait_stream(st)
        cur.synchronize()                                  # the caller holds the gradients on the host
        return sum(float(h[offs[4] + sizes[4]:offs[4] + sizes[4] + 4].view(torch.float32)[0]) for h in hout)   # dtemp
    e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        e2e_step()
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    h2d = P * chunk_bytes
    d2h = P * chunk_bytes

    # copies alone, both directions at once on two streams: the link's share of the end-to-end step on this host
    up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def copies_only():
        with torch.cuda.stream(up):
            for i in range(P):
                din[i].copy_(hin[i], non_blocking=True)
        with torch.cuda.stream(down):
            for i in range(P):
                hout[i].copy_(dout[i], non_blocking=True)
        up.synchronize(); down.synchronize()
    copies_only()
    barrier()
    t0 = time.perf_counter()
    for _ in range(3):
        copies_only()
    ms_copy = (time.perf_counter() - t0) / 3 * 1e3

    # strong scaling is the headline; the weak figure (64 sequences on every GPU) rides along when ranks > 1
    weak = None
    if dist_on and scaling == "strong" and not args.no_weak:
        del job
        torch.cuda.empty_cache()
        wjob = ScanJob(S, dev, GB, T, H, N, DK, DV, G, seed=rank, dist=args.dist)
        for _ in range(args.warmup):
            wjob.step()
        wms, _, _ = timed(wjob, args.steps, barrier)
        wms = max_over_ranks([wms], dev)[0]
        weak = {"value": whole_job_tokens_per_s(GB, T, world, args.steps, wms), "unit": "tokens/s",
                "ms_per_step": wms / args.steps, "global_batch": GB * world, "scaling": "weak"}
        del wjob
        torch.cuda.empty_cache()

    nseq = max_over_ranks([float(B)], dev)[0]
    ms, ms_e2e, ms_copy = max_over_ranks([ms, ms_e2e, ms_copy], dev)
    if rank == 0:
        toks = global_B * T * args.steps
        ab = algorithmic_bytes_per_token_head(N, DK, DV, G, 2, 2)
        peak, peak_kind = hbm_peak()
        # bytes each kernel is responsible for, per token and head (sums to ab["total"])
        # Snapshot rows >= 64 are zero-filled by a kernel on a second stream while the address scan runs (they are zero
        # for every sequence whose scan stays within 64 rows); the replay writes the rest.  Keys and values share one
        # launch when dk == dv.
        zf = min(N, 256 // max(DK // 8, 1))          # rows of the first row tile: everything above is zero-filled beside the scan
        kb_bytes = {"addr_fwd": 2 * DK * 2 + 8, "zero_fill": (N - zf) * (DK + DV) * 2 / G,
                    "replay_rows_k": zf * (DK + DV) * 2 / G + DV * 2, "replay_rows_v": 0,
                    "rows_bwd_k": (DK + DV) * 2 + N * (DK + DV) * 2 / G + (DK + DV) * 2, "rows_bwd_v": 0,
                    "addr_bwd": DK * 2 + 8 + DK * 2 + 8, "finish": 0}
        if DK != DV:     # keys and values then run as two launches
            kb_bytes["replay_rows_k"] = zf * DK * 2 / G
            kb_bytes["replay_rows_v"] = DV * 2 + zf * DV * 2 / G
            kb_bytes["rows_bwd_k"] = DK * 2 + N * DK * 2 / G + DK * 2
            kb_bytes["rows_bwd_v"] = DV * 2 + N * DV * 2 / G + DV * 2
        launches = sum(c for c, _ in prof.values())
        tot_ms = max(sum(x for _, x in prof.values()), 1e-9)
        kern = {}
        for n, (c, t) in prof.items():
            if not c:
                continue
            ms_l = t / c
            gbs = kb_bytes.get(n, 0) * B * T * H / (ms_l * 1e-3) / 1e9
            kern[n] = {"launches": c, "ms_per_launch": ms_l, "share": t / tot_ms,
                       "algorithmic_gbs": gbs, "frac_of_hbm_peak": gbs / peak}
        # The zero-fill runs BESIDE the address scan (two streams, same time window): for the roofline the pair counts as
        # one unit, its duration the longer of the two, its bytes the sum.
        units = {n: (prof[n][1] / max(prof[n][0], 1), kb_bytes.get(n, 0)) for n in prof if prof[n][0]}
        if "zero_fill" in units and "addr_fwd" in units:
            za, aa = units.pop("zero_fill"), units.pop("addr_fwd")
            units["addr_fwd||zero_fill"] = (max(za[0], aa[0]), za[1] + aa[1])
        top = max(units, key=lambda n: units[n][0])
        top_ms = units[top][0]
        top_bytes = units[top][1] * B * T * H
        achieved = top_bytes / (top_ms * 1e-3) / 1e9
        step_ms = ms / args.steps
        step_bytes = ab["total"] * H * B * T                              # per rank: ranks run side by side
        step_gbs = step_bytes / (step_ms * 1e-3) / 1e9
        traffic = None
        if top in NCU_TRAFFIC_B8 and T == SHAPE["T"] and args.dist == "bench":
            traffic = NCU_TRAFFIC_B8[top][0] * B / 8
        line = {"metric": METRIC, "value": toks / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": scaling,
                "vs_baseline": None, "dtype": "f32 state/accumulate, bf16 streams+snapshots", "data": "synthetic",
                "config": {"workload": "config1: slot-scan fwd+bwd, global B=%d (%d per GPU) T=%d H=%d N=%d dk=dv=%d G=%d, "
                                       "hard+detached, occ_bin, per-token fr, separate write query, dist=%s"
                                       % (global_B, int(nseq), T, H, N, DK, G, args.dist),
                           "global_batch": global_B, "seq_len": T, "sharding": "batch, no collective",
                           "l2": "working set %.1f GB per step and GPU >> 126 MB L2 (no flush needed)" % (step_bytes / 1e9)},
                "e2e": {"value": toks / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": ms_e2e / args.steps, "pipeline": "%d batch chunks on %d streams, one pinned staging buffer and one copy per chunk and direction" % (P, P),
                        "copies_only_ms": ms_copy, "copies_only_gbs_each_way": h2d / (ms_copy * 1e-3) / 1e9},
                "gpu_launches": launches,
                "roofline": {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak, "peak_kind": peak_kind, "traffic": traffic,
                             "traffic_source": NCU_TRAFFIC_B8[top][1] + " (B=8 capture scaled by B/8)" if traffic else None,
                             "algorithmic_bytes_per_launch": top_bytes,
                             "step": {"algorithmic_bytes": step_bytes, "achieved": step_gbs, "frac": step_gbs / peak}},
                "kernels": kern,
                "clocks": clocks}
        if weak is not None:
            line["weak"] = weak
        if world == 1:
            tb = job.touched_bytes()
            rf = line["roofline"]
            rf["touched_bytes_step"] = tb["step"]
            rf["touched_frac_step"] = tb["step"] / (step_ms * 1e-3) / 1e9 / peak
            rf["slots_used_mean"] = tb["slots_used_mean"]
            if top.startswith("rows_bwd"):
                rf["touched_bytes_per_launch"] = tb["rows_bwd"]
                rf["touched_frac"] = tb["rows_bwd"] / (top_ms * 1e-3) / 1e9 / peak
            if not args.no_extra:
                del job
                torch.cuda.empty_cache()
                if args.dist != "fill":
                    fjob = ScanJob(S, dev, B, T, H, N, DK, DV, G, seed=rank, dist="fill")
                    for _ in range(3):
                        fjob.step()
                    fms, fprof, _ = timed(fjob, max(3, args.steps // 2), barrier)
                    fsteps = max(3, args.steps // 2)
                    ftb = fjob.touched_bytes()
                    rf["fill"] = {"workload": "same shape, inputs that use every slot (dist=fill)", "ms_per_step": fms / fsteps,
                                  "value": B * T * fsteps / (fms * 1e-3), "unit": "tokens/s",
                                  "frac_step": step_bytes / (fms / fsteps * 1e-3) / 1e9 / peak,
                                  "touched_frac_step": ftb["step"] / (fms / fsteps * 1e-3) / 1e9 / peak,
                                  "slots_used_mean": ftb["slots_used_mean"],
                                  "kernels_ms": {n: t / c for n, (c, t) in fprof.items() if c}}
                    del fjob
                    torch.cuda.empty_cache()
                line["extra"] = {"reference_gpu_kernel": reference_kernel_leg(B, T, H, N, DK, G, 5, 3),
                                 "reference_gpu_kernel_fill": reference_kernel_leg(B, T, H, N, DK, G, 3, 2, dist="fill"),
                                 "read_bench": read_workload(args, local_rank, "bench"),
                                 "read_fill": read_workload(args, local_rank, "fill"),
                                 "epilogue": epilogue_workload(args, local_rank)}
            if not args.no_cpu:
                r = cpu_leg(3, 1, budget_s=30.0)
                line["cpu_baseline"] = {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port",
                                        "sample": r["sample"], "build": r["build"], "config0": r["config0"]}
        emit(line)
    if dist_on:
        dist.destroy_process_group()


def epilogue_workload(args, local_rank):
    """The writer epilogue + 3-bit storage quantiser over the snapshot tensors of the config-1 scan (keys with
    kinv / valid, then values), bf16 in, bf16 out.  One GPU; HBM-bound streaming."""
    import torch
    import slotscan_b200 as S
    torch.cuda.set_device(local_rank)
    B, T, H, N, D, G = (args.B or SHAPE["B"]), (args.T or SHAPE["T"]), SHAPE["H"], SHAPE["N"], SHAPE["DK"], SHAPE["G"]
    NB = (T + G - 1) // G
    g = torch.Generator(device="cuda").manual_seed(0)
    kbuf = torch.randn(B, NB, H, N, D, generator=g, device="cuda", dtype=torch.bfloat16)
    vbuf = torch.randn(B, NB, H, N, D, generator=g, device="cuda", dtype=torch.bfloat16)
    rows = kbuf.numel() // D
    out = {}
    for bits in (0, 3):
        for _ in range(3):
            S.writer_epilogue(kbuf, vbuf, torch.bfloat16, qbits=bits, qgroup=16)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            S.writer_epilogue(kbuf, vbuf, torch.bfloat16, qbits=bits, qgroup=16)
        b.record()
        torch.cuda.synchronize()
        out[bits] = a.elapsed_time(b) / args.steps
    peak, which = hbm_peak()
    # bits 0: keys are read, written and normed by the kernel; the values' cast bf16 -> bf16 is the identity (no pass)
    alg0 = rows * (2 * D * 2 + 5)
    alg3 = 2 * rows * 2 * D * 2 + rows * 5
    del kbuf, vbuf
    torch.cuda.empty_cache()
    return {"workload": "writer epilogue over (%d,%d,%d,%d,%d) bf16 keys and values" % (B, NB, H, N, D),
            "fq3_group16": {"ms": out[3], "achieved_gbs": alg3 / out[3] / 1e6, "frac": alg3 / out[3] / 1e6 / peak},
            "unquantised": {"ms": out[0], "achieved_gbs": alg0 / out[0] / 1e6, "frac": alg0 / out[0] / 1e6 / peak},
            "peak_source": which}


def read_workload(args, local_rank, dist):
    """One reader layer's cosine read (NQ = 2 queries per head) over the snapshots of the config-1 scan: scan -> writer
    epilogue once (untimed), then the read is timed, forward and backward, and beside it the reference's own read
    math (torch einsum + softmax, gqa25/memlm_sh.py:379-397) on the same device tensors."""
    import torch
    import slotscan_b200 as S
    torch.cuda.set_device(local_rank)
    s = SHAPE
    B, T, H, N, D, G, NQ = (args.B or s["B"]), (args.T or s["T"]), s["H"], s["N"], s["DK"], s["G"], 2
    inp = make_host_inputs(B, T, H, D, D, seed=0, dist=dist)
    k, q, v = (inp[n].cuda().to(torch.bfloat16) for n in ("k", "q", "v"))
    steps = max(3, args.steps // 2)

    def time_it(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    with torch.no_grad():
        kbuf, vbuf = S.kv_scan_g(k, v, inp["gate"].cuda(), inp["fr"].cuda(), N, 16.0, G=G, hard=True, detach_addr=True,
                                 q=q, occ_bin=True, out_dtype=torch.bfloat16)
        kq, vq, kinv, valid = S.writer_epilogue(kbuf, vbuf, torch.bfloat16)
        del kbuf, vbuf, k, q, v
        g = torch.Generator(device="cuda").manual_seed(1)
        qr = torch.randn(B, T, H, NQ, D, generator=g, device="cuda", dtype=torch.bfloat16)
        sharp = torch.nn.functional.softplus(torch.randn(B, T, H, NQ, generator=g, device="cuda")) + 1
        ms = time_it(lambda: S.read_snapshots(qr, sharp, kq, vq, kinv, valid, G))
        drd = torch.randn(B, T, H, NQ, D, generator=g, device="cuda", dtype=torch.bfloat16)
        v8 = valid.to(torch.uint8)
        ms_bwd = time_it(lambda: torch.ops.slotscan.read_bwd(qr, sharp, kq, vq, kinv, v8, drd, G))

        # the reference's read on the same tensors (library GEMMs + eager softmax), forward only
        NB = T // G

        def torch_read():
            qn = torch.nn.functional.normalize(qr.float(), dim=-1, eps=1e-6).to(qr.dtype)
            qb = qn.view(B, NB, G, H, NQ, D).permute(0, 1, 3, 2, 4, 5).reshape(B, NB, H, G * NQ, D)
            sc = torch.einsum("bjhmd,bjhnd->bjhmn", qb, kq).float() * kinv.unsqueeze(-2)
            sc = sc * sharp.view(B, NB, G, H, NQ).permute(0, 1, 3, 2, 4).reshape(B, NB, H, G * NQ, 1)
            att = torch.softmax(sc.masked_fill(~valid.unsqueeze(-2), float("-inf")), dim=-1).nan_to_num(0.0)
            return torch.einsum("bjhmn,bjhnd->bjhmd", att.to(vq.dtype), vq)
        ms_torch = time_it(torch_read) if T % G == 0 else None
    peak, which = hbm_peak()
    rows = kq.numel() // D
    alg = qr.numel() * 2 * 2 + sharp.numel() * 4 + 2 * rows * D * 2 + rows * 5      # q, rd, sharp, both snapshots, kinv+valid
    touched = qr.numel() * 2 * 2 + sharp.numel() * 4 + 2 * int(valid.sum()) * D * 2 + rows * 5
    bwd_bytes = touched + qr.numel() * 2 * 2 + sharp.numel() * 4 + 2 * rows * D * 2 + rows * 4
    out = {"workload": "cosine read of one reader layer: B=%d T=%d H=%d NQ=%d N=%d dk=dv=%d G=%d, dist=%s, valid rows per "
                       "snapshot %.1f of %d" % (B, T, H, NQ, N, D, G, dist, float(valid.sum()) / (rows / N), N),
           "fwd_ms": ms, "fwd_tokens_per_s": B * T / (ms * 1e-3),
           # invalid rows are masked out of the softmax and never loaded: the bytes that count are those of the valid
           # rows; the all-rows figure (what a dense batched GEMM reads) is given beside it
           "fwd_touched_gbs": touched / ms / 1e6, "fwd_touched_frac": touched / ms / 1e6 / peak,
           "fwd_all_rows_gbs": alg / ms / 1e6, "fwd_all_rows_frac": alg / ms / 1e6 / peak,
           "bwd_ms": ms_bwd, "bwd_gbs": bwd_bytes / ms_bwd / 1e6, "bwd_frac": bwd_bytes / ms_bwd / 1e6 / peak,
           "torch_reference_math_fwd_ms": ms_torch, "peak_source": which}
    del kq, vq, kinv, valid, qr, sharp, drd
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong: the global batch (64 sequences) is split over the GPUs; weak: 64 sequences per GPU")
    ap.add_argument("--B", type=int, default=0, help="sequences of the global batch (default 64)")
    ap.add_argument("--T", type=int, default=0, help="tokens per sequence (default 1024)")
    ap.add_argument("--dist", default="bench", help="input distribution: bench (the benchmark's) | fill (every slot used) | clustered")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the fill-distribution step and the read / epilogue figures")
    ap.add_argument("--no-weak", action="store_true", help="ranks > 1: skip the secondary weak-scaling figure")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="batch chunks (= streams) of the end-to-end leg")
    ap.add_argument("--workload", default="scan", choices=["scan", "epilogue", "read"],
                    help="scan: the headline fwd+bwd slot scan; epilogue / read: only that secondary figure (1 GPU)")
    args = ap.parse_args()
    claim_stdout()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)
    if args.workload == "epilogue":
        if rank == 0:
            emit(epilogue_workload(args, local_rank))
    elif args.workload == "read":
        if rank == 0:
            emit(read_workload(args, local_rank, args.dist))
    else:
        run_gpu(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
