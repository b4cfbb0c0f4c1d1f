"""GPU parity at the shapes the benchmark configurations name, against the CPU oracle.

  config 0   B=2, T=256, H=6, N=192, dk=dv=128, float32, forward: read vectors [B,T,H,128] through
             scan -> writer epilogue -> cosine read, and the final slot state
  config 1   B=64, T=1024, bf16: whole sequences cut out of the full-size forward + backward run
  config 2   the encoder memory (N=96) and the shared memory (N=192) back to back at the ends of the length
             curriculum, (B,T) = (512,128) and (64,1024), a few sequences each
Tolerances: float32 mode 1e-5 (reads, state); bf16 mode rtol = atol = 2e-3 on float32-typed results and the bf16
storage band (tests/scan_cases.py: bf16_band_report) on bf16-typed ones; addresses exact off the 1e-4 margin.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.scan_cases import address_report, allclose_report, bf16_band_report, make_inputs, rel_to_max

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _S():
    import slotscan_b200 as S
    return S


def test_config0_reads_and_final_state_fp32():
    """Config 0 at its exact shape and seed: outputs are the read vectors and the final slot state."""
    S = _S()
    B, T, H, N, D, G = 2, 256, 6, 192, 128, 8
    inp = make_inputs("bench", B, T, H, D, D, seed=0)
    gen = torch.Generator().manual_seed(1)
    qr = torch.randn(B, T, H, 1, D, generator=gen)
    qr = qr / qr.norm(dim=-1, keepdim=True)
    sharp = torch.nn.functional.softplus(torch.randn(B, T, H, 1, generator=gen)) + 1
    d = lambda x: x.to(DEV)
    with torch.no_grad():
        lg = S.scan_with_log(d(inp["k"]), d(inp["v"]), d(inp["gate"]), d(inp["fr"]), N, 16.0, G=G, q=d(inp["q"]),
                             occ_bin=True)
        kq, vq, kinv, valid = S.writer_epilogue(lg["kbuf"], lg["vbuf"], torch.float32)
        rd = S.read_snapshots(d(qr), d(sharp), kq, vq, kinv, valid, G)
    kw = dict(N=N, temp=16.0, G=G, hard=True, q=inp["q"], occ_bin=True)
    ref = O.scan_fwd(inp["k"], inp["v"], inp["gate"], inp["fr"], dtype=np.float64, **kw)
    ok, nflip, nbad, keep = address_report(lg["addr"].cpu().numpy(), ref["addr"], ref["margin"])
    print("config 0: address flips %d sequences of %d, beyond the 1e-4 margin %d; smallest oracle margin %.2e"
          % (nflip, B * H, nbad, ref["margin"].min()))
    assert ok and keep.all()
    ki_o, va_o = O.epilogue(ref["kbuf"])
    rd_o = O.read_fwd(qr.numpy(), sharp.numpy(), ref["kbuf"], ref["vbuf"], ki_o, va_o, G)
    assert np.array_equal(valid.cpu().numpy(), va_o)
    assert np.abs(rd.cpu().numpy() - rd_o).max() < 1e-5
    assert rd[:, :G].abs().max().item() == 0                           # block 0 reads the empty memory
    for n in ("kfin", "vfin", "ofin"):
        assert np.abs(lg[n].cpu().numpy().reshape(ref[n].shape) - ref[n]).max() < 1e-5, n


def _bf16_inputs(dist, B, T, H, D, seed):
    inp = make_inputs(dist, B, T, H, D, D, seed=seed)
    for n in ("k", "q", "v"):
        inp[n] = inp[n].to(torch.bfloat16)
    return inp


def _run_bf16(S, inp, N, G, dkb, dvb):
    """Forward + backward through the public call, bf16 streams and snapshots; returns outputs and the address log."""
    k, q, v = (inp[n].to(DEV).requires_grad_() for n in ("k", "q", "v"))
    g, fr = inp["gate"].to(DEV).requires_grad_(), inp["fr"].to(DEV).requires_grad_()
    tp = torch.tensor(16.0, device=DEV, requires_grad=True)
    kb, vb = S.kv_scan_g(k, v, g, fr, N, tp, G=G, hard=True, detach_addr=True, q=q, occ_bin=True,
                         out_dtype=torch.bfloat16)
    torch.autograd.backward([kb, vb], [dkb, dvb])
    with torch.no_grad():
        lg = S.scan_with_log(k.detach(), v.detach(), g.detach(), fr.detach(), N, 16.0, G=G, q=q.detach(), occ_bin=True,
                             out_dtype=torch.bfloat16)
    return dict(kbuf=kb.detach(), vbuf=vb.detach(), dk=k.grad, dq=q.grad, dv=v.grad, dgate=g.grad, dfr=fr.grad,
                addr=lg["addr"], kfin=lg["kfin"], vfin=lg["vfin"])


def _compare_sequences(tag, out, inp, dkb, dvb, N, G, H, seqs):
    """Whole sequences `seqs` of a batched bf16 run against the float64 oracle run on those sequences alone."""
    flips = 0
    for b in seqs:
        sl = slice(b, b + 1)
        one = {n: inp[n][sl].float() for n in ("k", "q", "v", "gate", "fr")}
        kw = dict(N=N, temp=16.0, G=G, hard=True, q=one["q"], occ_bin=True)
        ref = O.scan_fwd(one["k"], one["v"], one["gate"], one["fr"], dtype=np.float64, **kw)
        ok, nflip, nbad, keep = address_report(out["addr"][sl].cpu().numpy(), ref["addr"], ref["margin"])
        clear = ref["margin"].min(axis=1) > 1e-3
        print("%s sequence %d: heads with an address flip %d / %d (beyond the 1e-4 margin %d), smallest margin %.2e"
              % (tag, b, nflip, H, nbad, ref["margin"].min()))
        assert ok and keep[clear].all()
        flips += nflip
        wk, wv = dkb[sl].float().cpu().numpy(), dvb[sl].float().cpu().numpy()
        gr = O.scan_bwd(one["k"], one["v"], one["gate"], one["fr"], dkbuf=wk, dvbuf=wv, detach_addr=True,
                        dtype=np.float64, **kw)
        m5, m4, m3 = keep[:, None, :, None, None], keep[:, None, :, None], keep[:, None, :]
        for n in ("kbuf", "vbuf"):
            okc, worst, share = bf16_band_report(out[n][sl].float().cpu().numpy() * m5, ref[n] * m5)
            assert okc and share <= 5e-4, (tag, b, n, worst, share)
        for n in ("dk", "dq", "dv"):
            scale = max(np.abs(gr[n]).max(), 1e-30)
            okc, worst, share = bf16_band_report(out[n][sl].float().cpu().numpy() * m4, gr[n] * m4, scale)
            assert okc and share <= 5e-3, (tag, b, n, worst / scale, share)
        for n in ("dgate", "dfr"):
            scale = max(np.abs(gr[n]).max(), 1e-30)
            okc, worst = allclose_report(out[n][sl].cpu().numpy() * m3 / scale, gr[n] * m3 / scale, 2e-3, 2e-3)
            assert okc, (tag, b, n, worst)
        BH = slice(b * H, (b + 1) * H)
        for n in ("kfin", "vfin"):
            okc, worst = allclose_report(out[n][BH].cpu().numpy().reshape(ref[n].shape)[keep], ref[n][keep], 2e-3, 2e-3)
            assert okc, (tag, b, n, worst)
    return flips


def test_config1_full_size_sequences_vs_oracle():
    """The benchmark run itself (B=64, T=1024, H=6, N=192, D=128, G=8, bf16, forward + backward): the first, a middle
    and the last sequence of the batch against the oracle, values and gradients, not only properties."""
    S = _S()
    B, T, H, N, D, G = 64, 1024, 6, 192, 128, 8
    inp = _bf16_inputs("bench", B, T, H, D, seed=0)
    gen = torch.Generator(device=DEV).manual_seed(7)
    dkb = torch.randn(B, T // G, H, N, D, device=DEV, dtype=torch.bfloat16, generator=gen)
    dvb = torch.randn(B, T // G, H, N, D, device=DEV, dtype=torch.bfloat16, generator=gen)
    out = _run_bf16(S, inp, N, G, dkb, dvb)
    _compare_sequences("config 1", out, inp, dkb, dvb, N, G, H, (0, 31, 63))
    from slotscan_b200 import _lib
    assert _lib.device_status() == 0                                   # no kernel gave up on a bounded wait
    del out, dkb, dvb
    torch.cuda.empty_cache()


@pytest.mark.parametrize("BT", [(512, 128), (64, 1024)], ids=["B512_T128", "B64_T1024"])
def test_config2_two_memories_curriculum_ends(BT):
    """Config 2: the encoder memory (N=96) and the shared memory (N=192) written in the same pass, at both ends of
    the length curriculum (B*T = 65,536); three sequences of each run against the oracle."""
    S = _S()
    B, T = BT
    H, D, G = 6, 128, 8
    NB = (T + G - 1) // G
    for N, seed in ((96, 2), (192, 6)):                                 # layer 2 writes the encoder memory, layer 6 the shared one
        inp = _bf16_inputs("bench", B, T, H, D, seed=seed)
        gen = torch.Generator(device=DEV).manual_seed(11 + N)
        dkb = torch.randn(B, NB, H, N, D, device=DEV, dtype=torch.bfloat16, generator=gen)
        dvb = torch.randn(B, NB, H, N, D, device=DEV, dtype=torch.bfloat16, generator=gen)
        out = _run_bf16(S, inp, N, G, dkb, dvb)
        _compare_sequences("config 2 N=%d B=%d T=%d" % (N, B, T), out, inp, dkb, dvb, N, G, H, (0, B // 2, B - 1))
        del out, dkb, dvb
        torch.cuda.empty_cache()
