"""Runs the reference's OWN scan code (staged unmodified under baseline/_ref/gqa25/ by baseline/stage_reference.py) on a
seeded case and writes what it returns to an .npz file: a live check for the tests, beside the committed golden vectors.
  * `slotkern_kv._ref_scan_kv_impl` in float64 on the CPU (the definition, gqa25/slotkern_kv.py:66-123), snapshots and
    autograd gradients for seeded upstream weights;
  * with --cuda, also `slotkern_cuda.kv_scan_c` (the reference's production CUDA kernel, float32) on the GPU.
Inputs come from tests/scan_cases.make_inputs, the generator the parity tests use.  Runs in a process of its own
because the reference's module names (slotkern_cuda, slotkern_kvg, ...) are the names of this package's drop-in modules.

usage: python baseline/run_reference_scan.py OUT.npz dist B T H N DK DV G hard hard_gate occ_bin detach frtok sepq seed [--cuda]"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref", "gqa25")


def main():
    out_path, dist = sys.argv[1], sys.argv[2]
    B, T, H, N, DK, DV, G, hard, hard_gate, occ_bin, detach, frtok, sepq, seed = (int(x) for x in sys.argv[3:17])
    cuda = "--cuda" in sys.argv
    if "CUDA_HOME" not in os.environ and os.path.isdir("/usr/local/cuda/include"):
        os.environ["CUDA_HOME"] = "/usr/local/cuda"
    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.dirname(HERE))
    import numpy as np
    import torch
    from tests.scan_cases import make_inputs
    import slotkern_kv as KV
    assert os.path.dirname(os.path.abspath(KV.__file__)) == REF, KV.__file__
    torch.set_num_threads(8)
    inp = make_inputs(dist, B, T, H, DK, DV, seed=seed, frtok=bool(frtok), sepq=bool(sepq))
    d = lambda x: x.double().clone().requires_grad_()
    k, v, g, fr = d(inp["k"]), d(inp["v"]), d(inp["gate"]), d(inp["fr"])
    q = d(inp["q"]) if inp["q"] is not None else None
    tp = torch.tensor(float(inp["temp"]), dtype=torch.float64, requires_grad=True)
    pin = bool(hard) and not bool(detach)                  # see tests/golden/make_golden.py: the kernels' own definition there
    kb, vb, wb = KV._ref_scan_kv_impl(k, v, g, fr, N, tp, G=G, hard=bool(hard), hard_gate=bool(hard_gate), eps=1e-4,
                                      return_w=True, detach_addr=bool(detach), q=q, pin=pin, occ_bin=bool(occ_bin))
    gen = torch.Generator().manual_seed(seed + 1)
    wk, wv = torch.randn(kb.shape, generator=gen), torch.randn(vb.shape, generator=gen)
    ((kb * wk.double()).sum() + (vb * wv.double()).sum()).backward()
    out = dict(kbuf=kb.detach().numpy(), vbuf=vb.detach().numpy(), addr=wb.detach().argmax(-1).to(torch.int32).numpy(),
               wk=wk.numpy(), wv=wv.numpy(), dk=k.grad.numpy(), dv=v.grad.numpy(), dgate=g.grad.numpy(), dfr=fr.grad.numpy(),
               dtemp=tp.grad.numpy())
    if q is not None:
        out["dq"] = q.grad.numpy()
    if cuda:
        import slotkern_cuda as KC
        assert os.path.dirname(os.path.abspath(KC.__file__)) == REF, KC.__file__
        c = lambda x: x.float().cuda().requires_grad_()
        k2, v2, g2, fr2 = c(inp["k"]), c(inp["v"]), c(inp["gate"]), c(inp["fr"])
        q2 = c(inp["q"]) if inp["q"] is not None else None
        tp2 = torch.tensor(float(inp["temp"]), device="cuda", requires_grad=True)
        kb2, vb2 = KC.kv_scan_c(k2, v2, g2, fr2, N, tp2, G=G, hard=bool(hard), hard_gate=bool(hard_gate), detach_addr=bool(detach),
                                q=q2, occ_bin=bool(occ_bin))
        ((kb2 * wk.cuda()).sum() + (vb2 * wv.cuda()).sum()).backward()
        out.update(c_kbuf=kb2.detach().cpu().numpy(), c_vbuf=vb2.detach().cpu().numpy(), c_dk=k2.grad.cpu().numpy(),
                   c_dv=v2.grad.cpu().numpy(), c_dgate=g2.grad.cpu().numpy(), c_dfr=fr2.grad.cpu().numpy(),
                   c_dtemp=tp2.grad.cpu().numpy())
        if q2 is not None:
            out["c_dq"] = q2.grad.cpu().numpy()
    np.savez(out_path, **out)
    print("wrote", out_path)


if __name__ == "__main__":
    main()
