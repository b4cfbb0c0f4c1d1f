"""Times the reference's own CUDA scan, `slotkern_cuda.kv_scan_c` (runtime-compiled by torch's NVRTC wrapper; staged
unmodified under `baseline/_ref/gqa25/` by `baseline/stage_reference.py`), forward + backward on this GPU, with the
call the model makes (gqa25/memlm_sh.py:454-456: float32 streams, hard address, detached address gradient, per-token
fr, occ_bin) and the protocol of the reference's own timing script (kvu/bench_cuda.py:8-23: sum of both snapshot
tensors as the loss), but with CUDA events instead of wall clock.  Prints one JSON line.  Runs in its own process so
that the reference's modules never share an interpreter with this library.

usage: python baseline/time_reference_kernel.py B T H N D G steps warmup dist seed"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref", "gqa25")


def main():
    B, T, H, N, D, G, steps, warmup = (int(x) for x in sys.argv[1:9])
    dist, seed = sys.argv[9], int(sys.argv[10])
    if not os.path.isfile(os.path.join(REF, "slotkern_cuda.py")):
        print(json.dumps({"unavailable": "baseline/_ref/gqa25 is not staged"}))
        return
    if "CUDA_HOME" not in os.environ and os.path.isdir("/usr/local/cuda/include"):
        os.environ["CUDA_HOME"] = "/usr/local/cuda"
    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.dirname(HERE))
    import torch
    from tests.scan_cases import make_inputs                     # the same seeded inputs as this library's bench step
    import slotkern_cuda as KC                                   # the reference's module (first on sys.path)
    assert os.path.dirname(os.path.abspath(KC.__file__)) == REF, KC.__file__
    dev = "cuda"
    inp = make_inputs(dist, B, T, H, D, D, seed=seed)
    k, q, v, g, fr = (inp[n].to(dev, torch.float32).requires_grad_() for n in ("k", "q", "v", "gate", "fr"))
    temp = torch.tensor(float(inp["temp"]), device=dev, requires_grad=True)

    def fwd():
        return KC.kv_scan_c(k, v, g, fr, N, temp, G=G, hard=True, detach_addr=True, q=q, occ_bin=True)

    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    tf = tb = 0.0
    for it in range(warmup + steps):
        for t in (k, q, v, g, fr, temp):
            t.grad = None
        torch.cuda.synchronize()
        ev[0].record()
        kb, vb = fwd()
        ev[1].record()
        (kb.sum() + vb.sum()).backward()
        ev[2].record()
        torch.cuda.synchronize()
        if it >= warmup:
            tf += ev[0].elapsed_time(ev[1]) / steps
            tb += ev[1].elapsed_time(ev[2]) / steps
    attrs = {n: list(a) for n, a in KC.kernel_attrs(N, D, True, True, 1e-4).items()}
    print(json.dumps({"impl": "reference slotkern_cuda.kv_scan_c (NVRTC, float32 streams and snapshots)",
                      "fwd_ms": tf, "bwd_ms": tb, "step_ms": tf + tb, "tokens_per_s": B * T / (tf + tb) * 1e3,
                      "includes": "the loss (sum of both snapshot tensors) and its autograd expansion, as in kvu/bench_cuda.py",
                      "shape": dict(B=B, T=T, H=H, N=N, D=D, G=G), "dist": dist, "kernel_attrs_regs_local": attrs}))


if __name__ == "__main__":
    main()
