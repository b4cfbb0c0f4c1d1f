"""Benchmark of the slot-scan hot path: forward + backward of the hard-address scan at the sh25 training shape.

    python bench.py [--gpus N] [--steps K] [--warmup W]            this build's CUDA path
    python bench.py --impl reference [...]                          the CPU implementation timed on the host cores
    torchrun ... bench.py --gpus N ...                              one rank per GPU, batch-sharded (weak scaling)

One step = one forward + backward pass of the scan over one batch (B=64 sequences x T=1024 tokens x 6 heads per GPU,
N=192 slots, dk=dv=128, snapshot stride 8, bf16 token streams and snapshots, float32 state and accumulation), on
seeded synthetic inputs with the benchmark's distributions.  Prints ONE JSON line:
  value      tokens/s, whole job, inputs resident in HBM, device-timed (CUDA events, max over ranks)
  e2e        the same through the public Python API with HOST (pinned) inputs: H2D of k,q,v,gate,fr and D2H of every
             input gradient inside the timed region
  roofline   the dominant kernel's algorithmic bytes / its event-timed duration against the measured HBM peak
  cpu_baseline  the CPU oracle (C, OpenMP) on a bounded sample of the same workload, on this box's host cores
"""
import argparse
import json
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
    """Weak scaling: every rank scans its own B_per_rank sequences; the job's throughput counts all of them."""
    return B_per_rank * T * world * steps / (ms * 1e-3)


def make_host_inputs(B, T, H, DK, DV, seed, dist="bench"):
    from tests.scan_cases import make_inputs
    return make_inputs(dist, B, T, H, DK, DV, seed=seed)


# ------------------------------------------------------------------------------------------------------------------
def cpu_leg(steps, warmup, sample_B=2, threads=None, budget_s=90.0):
    """The CPU implementation of the same path: the C oracle (float32, OpenMP over (sequence, head)), forward + backward,
    on a bounded sample: `sample_B` sequences of the full T / H / N / D."""
    import numpy as np
    from oracle import oracle as O
    # all host cores the process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1 for its children)
    if not threads:
        try:
            threads = len(os.sched_getaffinity(0))
        except AttributeError:
            threads = os.cpu_count() or 1
    O.set_threads(threads)
    s = SHAPE
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
    steps = done
    toks = sample_B * s["T"] * steps
    return dict(value=toks / dt, ms_per_step=1e3 * dt / steps, cores=O.threads(), steps=steps,
                sample="%d of %d sequences, full T=%d H=%d N=%d D=%d G=%d, float32, fwd+bwd" %
                       (sample_B, s["B"], s["T"], s["H"], s["N"], s["DK"], s["G"]))


def run_reference(args, rank, world):
    if rank != 0:
        return
    warmup = min(args.warmup, 1)
    r = cpu_leg(max(1, args.steps), warmup)
    steps = r["steps"]
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config1: slot-scan fwd+bwd, B=64 T=1024 H=6 N=192 dk=dv=128 G=8 (CPU sample: see cpu_baseline.sample)",
                       "l2": "n/a (host)"},
            "cpu_baseline": {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]},
            "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


# ------------------------------------------------------------------------------------------------------------------
def run_gpu(args, rank, local_rank, world):
    import torch
    import slotscan_b200 as S
    from slotscan_b200 import _lib

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
    B, T, H, N, DK, DV, G = (s[n] for n in ("B", "T", "H", "N", "DK", "DV", "G"))
    NB = (T + G - 1) // G
    inp = make_host_inputs(B, T, H, DK, DV, seed=rank, dist=args.dist)       # each rank its own shard of the batch
    bf = torch.bfloat16
    host = {n: inp[n].to(bf).contiguous().pin_memory() for n in ("k", "q", "v")}
    host.update({n: inp[n].float().contiguous().pin_memory() for n in ("gate", "fr")})
    devin = {n: t.to(dev) for n, t in host.items()}
    temp = torch.tensor([16.0], device=dev)
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    dkb = torch.randn(B, NB, H, N, DK, device=dev, dtype=bf, generator=gen)
    dvb = torch.randn(B, NB, H, N, DV, device=dev, dtype=bf, generator=gen)

    def step(x):
        k, q, v = (x[n].detach().requires_grad_() for n in ("k", "q", "v"))
        g, fr = x["gate"].detach().requires_grad_(), x["fr"].detach().requires_grad_()
        tp = temp.detach().requires_grad_()
        kb, vb = S.kv_scan_g(k, v, g, fr, N, tp, G=G, hard=True, hard_gate=False, detach_addr=True, q=q, occ_bin=True,
                             out_dtype=bf)
        torch.autograd.backward([kb, vb], [dkb, dvb])
        return k.grad, q.grad, v.grad, g.grad, fr.grad, tp.grad

    def barrier():
        if dist_on:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(devin)
    barrier()
    # ---- device-timed leg: inputs resident in HBM ----
    _lib.profile_enable(True)
    _lib.profile_read()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clk:
        barrier()
        e0.record()
        for _ in range(args.steps):
            step(devin)
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    prof = _lib.profile_read()
    _lib.profile_enable(False)
    # ---- end-to-end leg: host inputs in, input gradients out, every step ----
    # The batch goes through in P chunks on P streams, so that the host->device copy of one chunk, the kernels of
    # another and the device->host copy of a third overlap (sequences are independent; the copies use both directions
    # of the link).  All through the public call, kv_scan_g, as a user would write it.
    P = args.e2e_chunks if B % args.e2e_chunks == 0 and B >= 2 * args.e2e_chunks else 1
    bs = B // P
    streams = [torch.cuda.Stream(device=dev) for _ in range(P)]
    hout = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (host["k"], host["q"], host["v"], host["gate"], host["fr"])]
    htemp = torch.empty(P, dtype=torch.float32).pin_memory()

    def e2e_step():
        cur = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(cur)
        for i, st in enumerate(streams):
            sl = slice(i * bs, (i + 1) * bs)
            st.wait_event(start)
            with torch.cuda.stream(st):
                x = {n: t[sl].to(dev, non_blocking=True) for n, t in host.items()}
                k, q, v = (x[n].requires_grad_() for n in ("k", "q", "v"))
                g, fr = x["gate"].requires_grad_(), x["fr"].requires_grad_()
                tp = temp.detach().requires_grad_()
                kb, vb = S.kv_scan_g(k, v, g, fr, N, tp, G=G, hard=True, hard_gate=False, detach_addr=True, q=q,
                                     occ_bin=True, out_dtype=bf)
                torch.autograd.backward([kb, vb], [dkb[sl], dvb[sl]])
                for h_, g_ in zip(hout, (k.grad, q.grad, v.grad, g.grad, fr.grad)):
                    h_[sl].copy_(g_, non_blocking=True)
                htemp[i:i + 1].copy_(tp.grad, non_blocking=True)
        for st in streams:
            cur.wait_stream(st)
        cur.synchronize()                                  # the caller holds the gradients on the host
        return float(htemp.sum())                          # dtemp is the sum over the chunks
    e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        e2e_step()
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = sum(t.numel() * t.element_size() for t in hout) + 4 * P
    ms, ms_e2e = max_over_ranks([ms, ms_e2e], dev)
    if rank == 0:
        toks = B * T * world * args.steps
        ab = algorithmic_bytes_per_token_head(N, DK, DV, G, 2, 2)
        peak, peak_kind = hbm_peak()
        # bytes each kernel is responsible for, per token and head (sums to ab["total"])
        kb_bytes = {"addr_fwd": 2 * DK * 2 + 8, "replay_rows_k": N * DK * 2 / G, "replay_rows_v": DV * 2 + N * DV * 2 / G,
                    "rows_bwd_k": (DK + DV) * 2 + N * (DK + DV) * 2 / G + (DK + DV) * 2, "rows_bwd_v": 0,
                    "addr_bwd": DK * 2 + 8 + DK * 2 + 8, "finish": 0}
        if DK != DV:     # keys and values then run as two launches
            kb_bytes["rows_bwd_k"] = DK * 2 + N * DK * 2 / G + DK * 2
            kb_bytes["rows_bwd_v"] = DV * 2 + N * DV * 2 / G + DV * 2
        launches = sum(c for c, _ in prof.values())
        tot_ms = max(sum(x for _, x in prof.values()), 1e-9)
        kern = {}
        for n, (c, t) in prof.items():
            if not c:
                continue
            ms_l = t / c
            gbs = kb_bytes[n] * B * T * H / (ms_l * 1e-3) / 1e9
            kern[n] = {"launches": c, "ms_per_launch": ms_l, "share": t / tot_ms,
                       "algorithmic_gbs": gbs, "frac_of_hbm_peak": gbs / peak}
        top = max(prof, key=lambda n: prof[n][1])
        top_ms = prof[top][1] / max(prof[top][0], 1)
        top_bytes = kb_bytes[top] * B * T * H
        achieved = top_bytes / (top_ms * 1e-3) / 1e9
        step_gbs = ab["total"] * H * B * T / (ms / args.steps * 1e-3) / 1e9
        line = {"metric": METRIC, "value": toks / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32 state/accumulate, bf16 streams+snapshots", "data": "synthetic",
                "config": {"workload": "config1: slot-scan fwd+bwd, B=%d/GPU T=%d H=%d N=%d dk=dv=%d G=%d, hard+detached, "
                                       "occ_bin, per-token fr, separate write query, dist=%s" % (B, T, H, N, DK, G, args.dist),
                           "global_batch": B * world, "seq_len": T, "sharding": "batch, no collective",
                           "l2": "working set %.1f GB per step >> 126 MB L2 (no flush needed)" % (ab["total"] * H * B * T / 1e9)},
                "e2e": {"value": toks / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": ms_e2e / args.steps, "pipeline": "%d batch chunks on %d streams" % (P, P)},
                "gpu_launches": launches,
                "roofline": {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak, "peak_kind": peak_kind, "traffic": TRAFFIC.get(top) if (B == SHAPE["B"] and T == SHAPE["T"] and args.dist == "bench") else None,
                             "algorithmic_bytes_per_launch": top_bytes,
                             "step": {"algorithmic_bytes": ab["total"] * H * B * T, "achieved": step_gbs, "frac": step_gbs / peak}},
                "kernels": kern,
                "clocks": clk.summary()}
        if world == 1 and not args.no_cpu:
            r = cpu_leg(1, 0)
            line["cpu_baseline"] = {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]}
        emit(line)
    if dist_on:
        dist.destroy_process_group()


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) at the benchmark size, from the ncu captures
# summarised under profiles/ (taken at B = 8 and scaled by 8: traffic is proportional to the batch)
# rows_bwd reads far fewer bytes than its algorithmic figure with the benchmark's inputs: snapshot-gradient rows of
# slots that were never candidates have no path to any input gradient and are skipped
TRAFFIC = {"replay_rows_k": 8 * (13.03e6 + 274.17e6), "replay_rows_v": 8 * (13.03e6 + 274.17e6), "addr_fwd": 8 * 25.6e6,
           "rows_bwd_k": 8 * (107.8e6 + 16.7e6), "addr_bwd": 8 * (52.34e6 + 0.96e6)}


def run_epilogue(args, local_rank):
    """Secondary line (`--workload epilogue`): the writer epilogue + 3-bit storage quantiser over the snapshots of the
    config-1 scan (keys with kinv / valid, then values), bf16 in, bf16 out.  One GPU; HBM-bound streaming."""
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
    with ClockSampler(local_rank) as clk:
        for bits in (0, 3):
            for _ in range(max(args.warmup, 3)):
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
    line = {"metric": "writer epilogue GB/s (config-1 snapshots, bf16)", "value": alg3 / out[3] / 1e6, "unit": "GB/s",
            "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": out[3],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 arithmetic on bf16 storage",
            "data": "synthetic", "gpu_launches": 2 * args.steps,
            "config": {"workload": "writer epilogue + _fq(3 bits, group 16) over (%d,%d,%d,%d,%d) keys and values"
                                   % (B, NB, H, N, D), "l2": "inputs (2 x %.1f GB) larger than L2" % (rows * D * 2 / 1e9)},
            "roofline": {"bound": "hbm", "achieved": alg3 / out[3] / 1e6, "peak": peak, "unit": "GB/s",
                         "frac": alg3 / out[3] / 1e6 / peak, "traffic": None, "peak_source": which},
            "unquantised": {"ms_per_step": out[0], "achieved": alg0 / out[0] / 1e6, "frac": alg0 / out[0] / 1e6 / peak},
            "clocks": clk.summary()}
    emit(line)


def run_read(args, local_rank):
    """Secondary line (`--workload read`): one reader layer's cosine read (NQ = 2 queries per head) over the snapshots of
    the config-1 scan: scan -> writer epilogue once (untimed), then the read is timed.  One GPU."""
    import torch
    import slotscan_b200 as S
    torch.cuda.set_device(local_rank)
    s = SHAPE
    B, T, H, N, D, G, NQ = (args.B or s["B"]), (args.T or s["T"]), s["H"], s["N"], s["DK"], s["G"], 2
    inp = make_host_inputs(B, T, H, D, D, seed=0, dist=args.dist)
    k, q, v = (inp[n].cuda().to(torch.bfloat16) for n in ("k", "q", "v"))
    with torch.no_grad():
        kbuf, vbuf = S.kv_scan_g(k, v, inp["gate"].cuda(), inp["fr"].cuda(), N, 16.0, G=G, hard=True, detach_addr=True,
                                 q=q, occ_bin=True, out_dtype=torch.bfloat16)
        kq, vq, kinv, valid = S.writer_epilogue(kbuf, vbuf, torch.bfloat16)
        g = torch.Generator(device="cuda").manual_seed(1)
        qr = torch.randn(B, T, H, NQ, D, generator=g, device="cuda", dtype=torch.bfloat16)
        sharp = torch.nn.functional.softplus(torch.randn(B, T, H, NQ, generator=g, device="cuda")) + 1
        with ClockSampler(local_rank) as clk:
            for _ in range(max(args.warmup, 3)):
                S.read_snapshots(qr, sharp, kq, vq, kinv, valid, G)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.steps):
                S.read_snapshots(qr, sharp, kq, vq, kinv, valid, G)
            b.record()
            torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        drd = torch.randn(B, T, H, NQ, D, generator=g, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            torch.ops.slotscan.read_bwd(qr, sharp, kq, vq, kinv, valid.to(torch.uint8), drd, G)
        torch.cuda.synchronize()
        a.record()
        for _ in range(args.steps):
            torch.ops.slotscan.read_bwd(qr, sharp, kq, vq, kinv, valid.to(torch.uint8), drd, G)
        b.record()
        torch.cuda.synchronize()
        ms_bwd = a.elapsed_time(b) / args.steps
    peak, which = hbm_peak()
    rows = kq.numel() // D
    alg = qr.numel() * 2 * 2 + sharp.numel() * 4 + 2 * rows * D * 2 + rows * 5      # q, rd, sharp, both snapshots, kinv+valid
    touched = qr.numel() * 2 * 2 + sharp.numel() * 4 + 2 * int(valid.sum()) * D * 2 + rows * 5
    line = {"metric": "snapshot read tokens/s per reader layer (config-1 shape, NQ=2, bf16)", "value": B * T / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 arithmetic on bf16 storage",
            "data": "synthetic", "gpu_launches": args.steps,
            "config": {"workload": "cosine read, forward: B=%d T=%d H=%d NQ=%d N=%d dk=dv=%d G=%d over the snapshots of the "
                                   "config-1 scan (dist=%s), valid rows per snapshot %.1f of %d"
                                   % (B, T, H, NQ, N, D, G, args.dist, float(valid.sum()) / (rows / N), N)},
            # invalid rows are masked out of the softmax and never loaded: the bytes that count are those of the valid
            # rows; the all-rows figure (what a dense batched GEMM reads) is given beside it
            "roofline": {"bound": "hbm", "achieved": touched / ms / 1e6, "peak": peak, "unit": "GB/s",
                         "frac": touched / ms / 1e6 / peak, "traffic": None, "peak_source": which,
                         "algorithmic_bytes": touched, "bytes_all_rows": alg, "achieved_all_rows": alg / ms / 1e6},
            # backward: re-reads what the forward read plus drd, writes dqr, dsharp and BOTH snapshot gradients in full
            # (exact zeros in the rows that are not valid) and dkinv
            "backward": {"ms_per_step": ms_bwd, "algorithmic_bytes": touched + qr.numel() * 2 * 2 + sharp.numel() * 4 + 2 * rows * D * 2 + rows * 4,
                         "achieved": (touched + qr.numel() * 2 * 2 + sharp.numel() * 4 + 2 * rows * D * 2 + rows * 4) / ms_bwd / 1e6,
                         "frac": (touched + qr.numel() * 2 * 2 + sharp.numel() * 4 + 2 * rows * D * 2 + rows * 4) / ms_bwd / 1e6 / peak},
            "clocks": clk.summary()}
    emit(line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--B", type=int, default=0, help="sequences per GPU (default 64)")
    ap.add_argument("--T", type=int, default=0, help="tokens per sequence (default 1024)")
    ap.add_argument("--dist", default="bench", help="input distribution: bench (the benchmark's) | fill (every slot used) | clustered")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="batch chunks (= streams) of the end-to-end leg")
    ap.add_argument("--workload", default="scan", choices=["scan", "epilogue", "read"],
                    help="scan: the headline fwd+bwd slot scan; epilogue: the writer epilogue + quantiser pass; "
                         "read: one reader layer's cosine read of the snapshots (secondary lines, 1 GPU)")
    args = ap.parse_args()
    claim_stdout()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.workload == "epilogue":
        if rank == 0:
            run_epilogue(args, local_rank)
    elif args.workload == "read":
        if rank == 0:
            run_read(args, local_rank)
    else:
        run_gpu(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
