"""Cosine read of the snapshots (CUDA, through the C ABI) against the reference's golden vector and the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _S():
    import slotscan_b200 as S
    return S


def rel(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max() / max(np.abs(b).max(), 1e-30))


def test_read_golden():
    S = _S()
    z = np.load(os.path.join(GOLDEN, "read_rsharp_nq2.npz"))
    G = int(z["G"])
    f = lambda n: torch.from_numpy(z[n].astype(np.float32)).cuda()
    with torch.no_grad():
        rd = S.read_snapshots(f("qr"), f("sharp"), f("kbuf"), f("vbuf"), f("kinv"), torch.from_numpy(z["valid"]).cuda(), G)
    assert rel(rd.cpu().numpy(), z["rd"]) < 1e-5                       # float32 mode tolerance
    assert rd[:, :G].abs().max() == 0                                  # block 0 reads the empty memory: exactly zero


def _case(B, T, H, NQ, N, DK, DV, G, nvalid, seed):
    g = torch.Generator().manual_seed(seed)
    NB = (T + G - 1) // G
    qr = torch.randn(B, T, H, NQ, DK, generator=g)
    sharp = torch.nn.functional.softplus(torch.randn(B, T, H, NQ, generator=g)) + 1
    kbuf = torch.randn(B, NB, H, N, DK, generator=g)
    vbuf = 0.5 * torch.randn(B, NB, H, N, DV, generator=g)
    # rows fill in index order as the scan proceeds: snapshot 0 is empty, the last one holds nvalid rows
    occ = torch.div(torch.arange(NB) * nvalid + max(NB - 2, 0), max(NB - 1, 1), rounding_mode="floor").clamp(max=nvalid).view(1, NB, 1, 1)
    live = torch.arange(N).view(1, 1, 1, N) < occ
    kbuf = kbuf * live.unsqueeze(-1)
    vbuf = vbuf * live.unsqueeze(-1)
    return qr, sharp, kbuf, vbuf


@pytest.mark.parametrize("shape", [(2, 40, 3, 2, 24, 128, 128, 8, 13), (1, 37, 2, 1, 192, 64, 64, 7, 192),
                                   (2, 16, 2, 4, 10, 16, 8, 16, 10), (1, 9, 1, 3, 70, 100, 36, 1, 40)],
                         ids=["sh25_like", "all_rows_T%G", "G16_NQ4_small", "G1_odd_widths"])
def test_read_matches_oracle_f32(shape):
    S = _S()
    B, T, H, NQ, N, DK, DV, G, nvalid = shape
    qr, sharp, kbuf, vbuf = _case(*shape, seed=5)
    kinv, valid = O.epilogue(kbuf.numpy(), dtype=np.float32)
    want = O.read_fwd(qr.numpy(), sharp.numpy(), kbuf.numpy(), vbuf.numpy(), kinv, valid, G, dtype=np.float64)
    with torch.no_grad():
        rd = S.read_snapshots(qr.cuda(), sharp.cuda(), kbuf.cuda(), vbuf.cuda(), torch.from_numpy(kinv).cuda(),
                              torch.from_numpy(valid).cuda(), G)
    assert rel(rd.cpu().numpy(), want) < 1e-5
    assert rd[:, :G].abs().max() == 0


def test_read_after_scan_and_epilogue_bf16():
    """The three ops in sequence as the writer and a reader layer use them: scan -> epilogue -> read, bf16 storage."""
    S = _S()
    from tests.scan_cases import make_inputs
    B, T, H, N, D, G, NQ = 2, 64, 3, 24, 32, 8, 2
    inp = make_inputs("bench", B, T, H, D, D, seed=7)
    k, q, v = (inp[n].cuda().to(torch.bfloat16) for n in ("k", "q", "v"))
    with torch.no_grad():
        kbuf, vbuf = S.kv_scan_g(k, v, inp["gate"].cuda(), inp["fr"].cuda(), N, 16.0, G=G, hard=True, detach_addr=True,
                                 q=q, occ_bin=True, out_dtype=torch.bfloat16)
        kq, vq, kinv, valid = S.writer_epilogue(kbuf, vbuf, torch.bfloat16)
        g = torch.Generator().manual_seed(8)
        qr = torch.randn(B, T, H, NQ, D, generator=g).cuda().to(torch.bfloat16)
        sharp = (torch.nn.functional.softplus(torch.randn(B, T, H, NQ, generator=g)) + 1).cuda()
        rd = S.read_snapshots(qr, sharp, kq, vq, kinv, valid, G)
    want = O.read_fwd(qr.float().cpu().numpy(), sharp.cpu().numpy(), kq.float().cpu().numpy(), vq.float().cpu().numpy(),
                      kinv.cpu().numpy(), valid.cpu().numpy(), G, dtype=np.float64)
    got = rd.float().cpu().numpy()
    # bf16 output: the oracle rounded to bf16, +- 1 ulp, plus the 2e-3 band of the bf16 mode
    assert np.all(np.abs(got - want) <= 2e-3 * np.abs(want).max() + np.abs(want) * 2.0 ** -7)
    assert rd.dtype == torch.bfloat16 and rd[:, :G].abs().max() == 0


@pytest.mark.parametrize("shape", [(2, 64, 3, 2, 192, 128, 128, 8, 192), (2, 40, 2, 2, 192, 128, 128, 8, 13),
                                   (1, 50, 2, 4, 96, 64, 64, 16, 96), (1, 21, 2, 1, 40, 128, 128, 8, 37),
                                   # the persistent ring kernel (G * NQ <= 16, N % 16 == 0): each box height, T % G != 0,
                                   # dk = 64, a short memory, M = 16 from NQ = 1, and more snapshots than SMs
                                   (2, 44, 2, 2, 192, 128, 128, 8, 100), (1, 64, 2, 2, 96, 64, 64, 8, 70),
                                   (1, 32, 2, 1, 192, 128, 128, 16, 50), (1, 30, 3, 2, 48, 128, 128, 4, 40),
                                   (4, 256, 6, 2, 192, 128, 128, 8, 150)],
                         ids=["sh25_dense", "sh25_sparse", "d64_M64_T%G", "M8_n40", "ring_box128_T%G", "ring_d64_n96",
                              "ring_box64_nq1", "ring_n48_m8", "ring_768_snapshots"])
def test_read_tensor_core_path_bf16(shape):
    """bf16 queries and snapshots with dk = dv in {64, 128}: the read runs on the tensor cores (Q K^T and P V as
    m16n8k16 MMAs with float32 accumulation, P in bf16 as the reference's att.to(bf16)).  Against the float64 oracle on
    the same bf16-rounded inputs, within the bf16 band: one bf16 ulp of the value plus 2e-3 of the tensor's scale."""
    S = _S()
    B, T, H, NQ, N, DK, DV, G, nvalid = shape
    qr, sharp, kbuf, vbuf = _case(*shape, seed=15)
    qr, kbuf, vbuf = (x.to(torch.bfloat16) for x in (qr, kbuf, vbuf))
    kinv, valid = O.epilogue(kbuf.float().numpy(), dtype=np.float32)
    want = O.read_fwd(qr.float().numpy(), sharp.numpy(), kbuf.float().numpy(), vbuf.float().numpy(), kinv, valid, G,
                      dtype=np.float64)
    with torch.no_grad():
        rd = S.read_snapshots(qr.cuda(), sharp.cuda(), kbuf.cuda(), vbuf.cuda(), torch.from_numpy(kinv).cuda(),
                              torch.from_numpy(valid).cuda(), G)
    got = rd.float().cpu().numpy()
    assert rd.dtype == torch.bfloat16 and rd[:, :G].abs().max() == 0
    assert np.all(np.abs(got - want) <= 2e-3 * np.abs(want).max() + np.abs(want) * 2.0 ** -7), \
        float((np.abs(got - want) - np.abs(want) * 2.0 ** -7).max() / np.abs(want).max())
    # mean error far inside the band: the kernel is not merely "within an ulp" everywhere
    assert np.abs(got - want).mean() < 2e-3 * np.abs(want).max()
    from slotscan_b200 import _lib
    assert _lib.device_status() == 0


def test_read_contract():
    S = _S()
    qr, sharp, kbuf, vbuf = _case(1, 8, 1, 1, 4, 16, 16, 4, 4, seed=1)
    kinv, valid = O.epilogue(kbuf.numpy(), dtype=np.float32)
    ki, va = torch.from_numpy(kinv), torch.from_numpy(valid)
    with pytest.raises(RuntimeError):
        S.read_snapshots(qr, sharp, kbuf, vbuf, ki, va, 4)            # CPU tensors
    with pytest.raises(ValueError):
        S.read_snapshots(qr.cuda(), sharp.cuda(), kbuf.cuda(), vbuf.cuda(), ki.cuda(), va.cuda(), 3)   # NB mismatch


def test_read_backward_golden():
    """Gradients of the read against the reference's autograd (golden vector): kinv is computed from kbuf under
    autograd there, so the chain here is writer_epilogue -> read_snapshots."""
    S = _S()
    z = np.load(os.path.join(GOLDEN, "read_rsharp_nq2.npz"))
    G = int(z["G"])
    f = lambda n: torch.from_numpy(z[n].astype(np.float32)).cuda()
    qr, sharp = f("qr").requires_grad_(), f("sharp").requires_grad_()
    kbuf, vbuf = f("kbuf").requires_grad_(), f("vbuf").requires_grad_()
    kq, vq, kinv, valid = S.writer_epilogue(kbuf, vbuf, torch.float32)
    rd = S.read_snapshots(qr, sharp, kq, vq, kinv, valid, G)
    rd.backward(f("drd"))
    assert rel(qr.grad.cpu().numpy(), z["dqr"]) < 1e-5
    assert rel(vbuf.grad.cpu().numpy(), z["dvbuf"]) < 1e-5
    assert rel(kbuf.grad.cpu().numpy(), z["dkbuf"]) < 1e-5
    C = float(z["C"])
    ds_raw = sharp.grad.cpu().numpy() * z["sharp"] * (1 - np.tanh(z["s_raw"].reshape(z["sharp"].shape) / C) ** 2)
    assert rel(ds_raw.reshape(z["ds_raw"].shape), z["ds_raw"]) < 1e-5


@pytest.mark.parametrize("shape", [(2, 40, 3, 2, 24, 128, 128, 8, 13), (1, 37, 2, 1, 192, 64, 64, 7, 192),
                                   (2, 16, 2, 4, 10, 16, 8, 16, 10), (1, 9, 1, 3, 70, 100, 36, 1, 40)],
                         ids=["sh25_like", "all_rows_T%G", "G16_NQ4_small", "G1_odd_widths"])
def test_read_backward_matches_oracle(shape):
    S = _S()
    B, T, H, NQ, N, DK, DV, G, nvalid = shape
    qr, sharp, kbuf, vbuf = _case(*shape, seed=6)
    drd = torch.randn(B, T, H, NQ, DV, generator=torch.Generator().manual_seed(9))
    kinv, valid = O.epilogue(kbuf.numpy(), dtype=np.float64)
    want = O.read_bwd(qr.numpy(), sharp.numpy(), kbuf.numpy(), vbuf.numpy(), kinv, valid, G, drd.numpy(),
                      kinv_const=True, dtype=np.float64)
    dqr, dsharp, dkbuf, dvbuf, dkinv = torch.ops.slotscan.read_bwd(
        qr.cuda(), sharp.cuda(), kbuf.cuda(), vbuf.cuda(), torch.from_numpy(kinv).float().cuda(),
        torch.from_numpy(valid).cuda(), drd.cuda(), G)
    assert rel(dqr.cpu().numpy(), want["dqr"]) < 1e-5
    assert rel(dsharp.cpu().numpy(), want["dsharp"]) < 1e-5
    assert rel(dvbuf.cpu().numpy(), want["dvbuf"]) < 1e-5
    assert rel(dkbuf.cpu().numpy(), want["dkbuf"]) < 1e-5
    # the kinv path: oracle with kinv differentiated = direct part + dkinv * d kinv / d kbuf
    full = O.read_bwd(qr.numpy(), sharp.numpy(), kbuf.numpy(), vbuf.numpy(), kinv, valid, G, drd.numpy(),
                      kinv_const=False, dtype=np.float64)
    mine = dkbuf.cpu().double().numpy() + (dkinv.cpu().double().numpy() * -(kinv ** 3))[..., None] * kbuf.double().numpy() * valid[..., None]
    assert rel(mine, full["dkbuf"]) < 1e-5
    # rows that are not valid get exact zeros; repeatable bit for bit
    assert (dkbuf.cpu()[~torch.from_numpy(valid)] == 0).all() and (dvbuf.cpu()[~torch.from_numpy(valid)] == 0).all()
    again = torch.ops.slotscan.read_bwd(qr.cuda(), sharp.cuda(), kbuf.cuda(), vbuf.cuda(), torch.from_numpy(kinv).float().cuda(),
                                        torch.from_numpy(valid).cuda(), drd.cuda(), G)
    assert all(torch.equal(a, b) for a, b in zip(again, (dqr, dsharp, dkbuf, dvbuf, dkinv)))


@pytest.mark.parametrize("shape", [(2, 44, 2, 2, 192, 128, 128, 8, 100), (1, 64, 2, 2, 96, 64, 64, 8, 70),
                                   (1, 32, 2, 1, 192, 128, 128, 16, 50), (4, 256, 6, 2, 192, 128, 128, 8, 150),
                                   (1, 64, 3, 2, 192, 128, 128, 8, 192)],
                         ids=["box128_T%G", "d64_n96", "box64_nq1", "768_snapshots", "all_rows"])
def test_read_backward_tensor_core_path_bf16(shape):
    """bf16 queries, snapshots and upstream gradient with dk = dv in {64, 128}: snapshots with more than 32 rows in use
    take the tensor-core backward (five MMAs per snapshot, att and G in bf16, float32 accumulation, snapshot gradients
    leave by tiled bulk tensor stores), the others the CUDA-core kernel.  Against the float64 oracle on the same
    bf16-rounded inputs: bf16-typed gradients within 6e-3 of their max (one bf16 rounding of att / G per term plus the
    rounding of the result; measured 2e-3 .. 4e-3), the float32-typed ones (dsharp, dkinv) within 1e-5 (measured 3e-7); rows
    that are not valid exactly zero."""
    S = _S()
    B, T, H, NQ, N, DK, DV, G, nvalid = shape
    qr, sharp, kbuf, vbuf = _case(*shape, seed=21)
    drd = torch.randn(B, T, H, NQ, DV, generator=torch.Generator().manual_seed(22))
    qr, kbuf, vbuf, drd = (x.to(torch.bfloat16) for x in (qr, kbuf, vbuf, drd))
    kinv, valid = O.epilogue(kbuf.float().numpy(), dtype=np.float32)
    f64 = lambda x: x.float().numpy().astype(np.float64)
    want = O.read_bwd(f64(qr), sharp.numpy(), f64(kbuf), f64(vbuf), kinv, valid, G, f64(drd), kinv_const=True, dtype=np.float64)
    args = (qr.cuda(), sharp.cuda(), kbuf.cuda(), vbuf.cuda(), torch.from_numpy(kinv).cuda(), torch.from_numpy(valid).cuda(),
            drd.cuda(), G)
    dqr, dsharp, dkbuf, dvbuf, dkinv = torch.ops.slotscan.read_bwd(*args)
    assert dqr.dtype == torch.bfloat16 and dkbuf.dtype == torch.bfloat16 and dvbuf.dtype == torch.bfloat16
    errs = {n: rel(g.float().cpu().numpy(), want[n]) for n, g in (("dqr", dqr), ("dkbuf", dkbuf), ("dvbuf", dvbuf), ("dsharp", dsharp))}
    # dkinv against the oracle: d kbuf with kinv differentiated minus the direct part, divided out row by row
    full = O.read_bwd(f64(qr), sharp.numpy(), f64(kbuf), f64(vbuf), kinv, valid, G, f64(drd), kinv_const=False, dtype=np.float64)
    kb = f64(kbuf)
    chain = (full["dkbuf"] - want["dkbuf"])                                  # = dkinv * (-kinv^3) * kbuf on valid rows
    dkinv_want = (chain * kb).sum(-1) / np.maximum((kb * kb).sum(-1), 1e-30) / -(kinv.astype(np.float64) ** 3) * valid
    errs["dkinv"] = rel(dkinv.cpu().numpy(), dkinv_want)
    print(shape, {n: "%.1e" % e for n, e in errs.items()})
    for n in ("dqr", "dkbuf", "dvbuf"):
        assert errs[n] < 6e-3, (n, errs[n])
    assert errs["dsharp"] < 1e-5 and errs["dkinv"] < 1e-5, errs
    inval = ~torch.from_numpy(valid.astype(bool))
    assert (dkbuf.cpu()[inval] == 0).all() and (dvbuf.cpu()[inval] == 0).all() and (dkinv.cpu()[inval] == 0).all()
    again = torch.ops.slotscan.read_bwd(*args)
    assert all(torch.equal(a, b) for a, b in zip(again, (dqr, dsharp, dkbuf, dvbuf, dkinv)))       # repeatable bit for bit
    from slotscan_b200 import _lib
    assert _lib.device_status() == 0
