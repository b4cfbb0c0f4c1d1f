"""Generates the golden fixtures of this directory by RUNNING THE REFERENCE's own torch code on CPU.

Needs the reference checkout, its location given in $SLOTSCAN_REFERENCE; it imports, unmodified,
    gqa25/slotkern_kv.py   _ref_scan_kv_impl / ref_scan_kv     (the scan; gradients by torch autograd)
    gqa25/memlm_sh.py      SharedMixer._read, _fq, _quantize_mem (the read and the storage quantiser)
    gqa25/slotkern_v.py    ref_scan_v                          (the keyless scan)
and writes one compressed .npz per case.  The fixtures travel with the repository; the reference does not.

    SLOTSCAN_REFERENCE=<reference checkout> python tests/golden/make_golden.py      # rewrites tests/golden/*.npz

Case list follows the reference's own test protocols: gqa25/test_kvg.py:6-12 (soft, attached/detached, T % G != 0,
separate query, G = 1), gqa25/test_frtok.py:13-36 (clustered keys, per-token fr, fr/temp in [0.2, 1.5]),
kvu/test_cuda.py:11-26 (hard + detached, gates forced to exact 0/1, hard gate, N not a multiple of anything),
gqa25/hardcheck.py:8-19 (k = 0.3 randn, g = sigmoid(randn - 0.5), fr 4.48), and the seeded distributions of the
benchmark configuration (unit keys, 0.5 randn values, sigmoid gates, fr = 0.1 randn, independent unit write query).
"""
import os
import sys
import types

import numpy as np
import torch

REF = os.environ.get("SLOTSCAN_REFERENCE")
if not REF or not os.path.isdir(os.path.join(REF, "gqa25")):
    sys.exit("make_golden.py: set SLOTSCAN_REFERENCE to the reference checkout (the directory that holds gqa25/)")
sys.path.insert(0, os.path.join(REF, "gqa25"))
HERE = os.path.dirname(os.path.abspath(__file__))

import slotkern_kv as KV  # noqa: E402  (the reference)


def clustered(gen, B, T, H, D, ncl, noise):
    cen = torch.randn(B, ncl, H, D, generator=gen)
    idx = torch.randint(0, ncl, (B, T), generator=gen)
    x = torch.gather(cen, 1, idx[:, :, None, None].expand(B, T, H, D))
    return x + noise * torch.randn(B, T, H, D, generator=gen)


def unit(x):
    return x / x.norm(dim=-1, keepdim=True)


SCAN_CASES = [
    # name, B, T, H, N, DK, DV, G, hard, hard_gate, occ_bin, detach, frtok, sepq, dist
    ("soft_attached", 2, 50, 3, 12, 8, 8, 16, 0, 0, 0, 0, 0, 0, "plain"),
    ("soft_detached", 2, 50, 3, 12, 8, 8, 16, 0, 0, 0, 1, 0, 0, "plain"),
    ("soft_attached_q_g7", 1, 64, 2, 24, 16, 16, 7, 0, 0, 0, 0, 0, 1, "plain"),
    ("soft_detached_g1", 1, 40, 2, 10, 8, 8, 1, 0, 0, 0, 1, 0, 0, "plain"),
    ("soft_occbin_frtok_clustered", 2, 50, 3, 12, 8, 8, 16, 0, 0, 1, 1, 1, 1, "clustered"),
    ("soft_frtok_attached_clustered", 2, 50, 3, 12, 8, 8, 16, 0, 0, 0, 0, 1, 1, "clustered"),
    ("hard_detached_occbin_frtok_clustered", 2, 96, 2, 16, 16, 16, 8, 1, 0, 1, 1, 1, 1, "clustered"),
    ("hard_detached_gates01", 1, 120, 2, 40, 32, 32, 16, 1, 0, 0, 1, 0, 0, "gates01"),
    ("hard_detached_hardgate_g7", 1, 70, 2, 40, 32, 32, 7, 1, 1, 1, 1, 0, 1, "gates01"),
    ("hard_detached_n50_d64", 1, 64, 1, 50, 64, 64, 8, 1, 0, 0, 1, 0, 1, "gates01"),
    ("hard_attached_hardcheck", 1, 64, 2, 16, 16, 16, 4, 1, 0, 0, 0, 0, 0, "hardcheck"),
    ("hard_bench_dist_d128", 1, 48, 1, 16, 128, 128, 8, 1, 0, 1, 1, 1, 1, "bench"),
    ("hard_bench_dist_dk_ne_dv", 1, 40, 2, 12, 32, 16, 8, 1, 0, 1, 1, 1, 1, "bench"),
]


def scan_inputs(gen, B, T, H, DK, DV, frtok, sepq, dist):
    # every input is drawn and shaped in float32, then widened: the float64 reference and a float32 kernel
    # see exactly the same numbers, and the fixture stores them losslessly as float32
    r = lambda *s: torch.randn(*s, generator=gen)
    u = lambda *s: torch.rand(*s, generator=gen)
    temp = 16.0
    if dist == "plain":                                   # gqa25/test_kvg.py:14-20
        k, q, v, g = r(B, T, H, DK), (r(B, T, H, DK) if sepq else None), r(B, T, H, DV), u(B, T, H)
        fr = temp * (0.2 + 1.3 * u(B, T, H)) if frtok else torch.tensor([2.0])
    elif dist == "clustered":                             # gqa25/test_frtok.py:31-36
        k = clustered(gen, B, T, H, DK, 6, 0.3)
        q = k + 0.2 * r(B, T, H, DK) if sepq else None
        v, g = r(B, T, H, DV), u(B, T, H)
        fr = temp * (0.2 + 1.3 * u(B, T, H)) if frtok else torch.tensor([9.0])
    elif dist == "gates01":                               # kvu/test_cuda.py:21-28
        k, q, v = r(B, T, H, DK), (r(B, T, H, DK) if sepq else None), r(B, T, H, DV)
        g, m = u(B, T, H), u(B, T, H)
        g = torch.where(m < 0.15, torch.zeros_like(g), torch.where(m > 0.92, torch.ones_like(g), g))
        fr = 2 * u(B, T, H) if frtok else torch.tensor([1.5])
    elif dist == "hardcheck":                             # gqa25/hardcheck.py:8-13
        k, q, v = 0.3 * r(B, T, H, DK), None, r(B, T, H, DV)
        g = torch.sigmoid(r(B, T, H) - 0.5)
        fr = torch.tensor([4.48])
    elif dist == "bench":                                 # the seeded benchmark distributions
        k, v = unit(r(B, T, H, DK)), 0.5 * r(B, T, H, DV)
        g, fr = torch.sigmoid(r(B, T, H)), 0.1 * r(B, T, H)
        q = unit(r(B, T, H, DK))
    else:
        raise ValueError(dist)
    d = lambda x: None if x is None else x.float().double()
    return d(k), d(q), d(v), d(g), d(fr), temp


def has_faint_rows(k, q, v, g, fr, temp, N, hard, hard_gate, occ_bin):
    """True if some row ever holds a key with 0 < |K| < 1e-6 (written, yet under the norm clamp)."""
    with torch.no_grad():
        kb, _ = KV._ref_scan_kv_impl(k, v, g, fr, N, torch.tensor(temp, dtype=torch.float64), G=1, hard=bool(hard),
                                     hard_gate=bool(hard_gate), q=q, pin=False, occ_bin=bool(occ_bin))
    nk = kb.norm(dim=-1)
    return bool(((nk > 0) & (nk < 1e-6)).any())


def make_scan_case(name, B, T, H, N, DK, DV, G, hard, hard_gate, occ_bin, detach, frtok, sepq, dist, seed):
    while True:
        gen = torch.Generator().manual_seed(seed)
        k, q, v, g, fr, temp = scan_inputs(gen, B, T, H, DK, DV, frtok, sepq, dist)
        # ATTACHED address only: where a written row sits under the 1e-6 norm clamp, torch autograd differentiates
        # K / clamp (gain 1e6) while the kernels define the match gradient as zero (gqa25/slotkern_kvg.py:187-188).
        # The two are different functions there, so attached fixtures use a seed on which no such row occurs.
        if detach or not has_faint_rows(k, q, v, g, fr, temp, N, hard, hard_gate, occ_bin):
            break
        seed += 1000
    leaves = {n: x.clone().requires_grad_() for n, x in dict(k=k, v=v, gate=g, fr=fr).items()}
    if q is not None:
        leaves["q"] = q.clone().requires_grad_()
    tp = torch.tensor(temp, dtype=torch.float64, requires_grad=True)
    # pin=False is the function the kernels compute (gqa25/slotkern_kv.py:94-99).  One exception: with a HARD and
    # ATTACHED address torch autograd sends the first free (all-zero) row's match gradient through the 1e-6 norm
    # clamp, a gain of 1e6 per step that overflows within tens of tokens (slotkern_kv.py:88-93).  The kernels zero
    # that term where the norm is clamped (gqa25/slotkern_kvg.py:187-188); pin=True does the same to the autograd
    # graph and leaves the forward unchanged here (no row with 0 < |K| < 1e-6 in this case).
    pin = bool(hard) and not bool(detach)
    kb, vb, wb = KV._ref_scan_kv_impl(leaves["k"], leaves["v"], leaves["gate"], leaves["fr"], N, tp, G=G, hard=bool(hard),
                                      hard_gate=bool(hard_gate), eps=1e-4, return_w=True, detach_addr=bool(detach),
                                      q=leaves.get("q"), pin=pin, occ_bin=bool(occ_bin))
    wk = torch.randn(kb.shape, generator=gen).double()
    wv = torch.randn(vb.shape, generator=gen).double()
    ((kb * wk).sum() + (vb * wv).sum()).backward()
    f32 = lambda x: x.float()
    out = dict(k=f32(k), v=f32(v), gate=f32(g), fr=f32(fr), temp=np.float64(temp), kbuf=kb.detach(), vbuf=vb.detach(),
               addr=wb.detach().argmax(-1).to(torch.int32), addr_w=f32(wb.detach()), wk=f32(wk), wv=f32(wv), dk=leaves["k"].grad, dv=leaves["v"].grad, dgate=leaves["gate"].grad,
               dfr=leaves["fr"].grad, dtemp=tp.grad,
               meta=np.array([B, T, H, N, DK, DV, G, hard, hard_gate, occ_bin, detach, frtok, sepq], np.int64))
    if q is not None:
        out["q"] = f32(q)
        out["dq"] = leaves["q"].grad
    # the same case through the fp32 public wrapper (what a model on CPU runs): forward only
    with torch.no_grad():
        kb32, vb32 = KV.ref_scan_kv(k.float(), v.float(), g.float(), fr.float(), N, torch.tensor(temp), G=G, hard=bool(hard),
                                    hard_gate=bool(hard_gate), detach_addr=bool(detach), q=None if q is None else q.float(),
                                    pin=False, occ_bin=bool(occ_bin))
    out["kbuf_f32"], out["vbuf_f32"] = kb32, vb32
    if hard:
        del out["addr_w"]                                  # one-hot: the int32 address says it all
    np.savez_compressed(os.path.join(HERE, "scan_%s.npz" % name),
                        **{n: (x.numpy() if torch.is_tensor(x) else x) for n, x in out.items()})
    print("scan_%s.npz  kbuf %s" % (name, tuple(kb.shape)))


def make_read_case(seed=11):
    """SharedMixer._read on scan output, with per-token read sharpness (sh_rsharp) and NQ = 2, T % G != 0."""
    import memlm_sh as S                                   # the reference model file
    gen = torch.Generator().manual_seed(seed)
    B, T, Hs, NQ, N, dk, dv, G, C = 2, 21, 3, 2, 10, 16, 8, 4, 2.0
    r = lambda *s: torch.randn(*s, dtype=torch.float64, generator=gen)
    k, v, g = r(B, T, Hs, dk), r(B, T, Hs, dv), torch.rand(B, T, Hs, dtype=torch.float64, generator=gen)
    kb, vb = KV._ref_scan_kv_impl(k, v, g, torch.tensor([2.0], dtype=torch.float64), N, torch.tensor(16.0, dtype=torch.float64),
                                  G=G, hard=True, detach_addr=True, pin=False, occ_bin=True)
    kb = kb.clone().requires_grad_()
    vb = vb.clone().requires_grad_()
    nsq = kb.pow(2).sum(-1)
    kinv, valid = torch.rsqrt(nsq.clamp_min(1e-12)), nsq > 1e-12
    x = r(B, T, Hs * NQ * dk).requires_grad_()             # tk_q is the identity here: x IS the raw read query
    s_raw = r(B, T, Hs * NQ).requires_grad_()
    log_rsel = torch.tensor(np.log(8.0), dtype=torch.float64)
    fake = types.SimpleNamespace(Hs=Hs, NQ=NQ, dk=dk, dv=dv, G=G, pos=0, tk_q=lambda z: z, log_rsel=log_rsel,
                                 _rsq=[lambda z: s_raw], rsharp=C, rs_a=None)
    rd = S.SharedMixer._read(fake, kb, vb, kinv, valid, x)          # (B,T,Hs,NQ,dv)
    drd = r(*rd.shape)
    (rd * drd).sum().backward()
    sharp = torch.exp(log_rsel + C * torch.tanh(s_raw.detach() / C)).reshape(B, T, Hs, NQ)
    np.savez_compressed(os.path.join(HERE, "read_rsharp_nq2.npz"),
                        qr=x.detach().reshape(B, T, Hs, NQ, dk).numpy(), sharp=sharp.numpy(), s_raw=s_raw.detach().numpy(),
                        C=np.float64(C), kbuf=kb.detach().numpy(), vbuf=vb.detach().numpy(), kinv=kinv.detach().numpy(),
                        valid=valid.numpy(), rd=rd.detach().numpy(), drd=drd.numpy(),
                        dqr=x.grad.reshape(B, T, Hs, NQ, dk).numpy(), ds_raw=s_raw.grad.numpy(),
                        dkbuf=kb.grad.numpy(), dvbuf=vb.grad.numpy(), G=np.int64(G))
    print("read_rsharp_nq2.npz  rd", tuple(rd.shape))


def make_quant_case(seed=3):
    """_fq at every supported width and two group sizes, plus _quantize_mem's kinv / valid."""
    import memlm_sh as S
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(2, 5, 3, 7, 64, generator=gen)
    x[0, 0, 0, 0] = 0.0                                    # a never-written row (gqa25/test_sh.py:97)
    x[1, 2, 1, 3, :16] = 0.0                               # one all-zero group inside a written row
    out = dict(x=x.numpy())
    for bits in (2, 3, 4, 8):
        for group in (16, 64):
            out["fq_b%d_g%d" % (bits, group)] = S._fq(x, bits, group).numpy()
    kq, vq, kinv, valid = S._quantize_mem(x, x * 0.5, 3, 16)
    out.update(qm_k=kq.numpy(), qm_v=vq.numpy(), qm_kinv=kinv.numpy(), qm_valid=valid.numpy())
    np.savez_compressed(os.path.join(HERE, "quant_fq.npz"), **out)
    print("quant_fq.npz")


KEYLESS_CASES = [   # name, B, T, H, N, DV, G, hard, hard_gate      (the self-test of gqa25/slotkern_v.py:283-289)
    ("soft_g1", 2, 40, 2, 12, 8, 1, 0, 0),
    ("hard_g4", 2, 50, 2, 16, 16, 4, 1, 0),
    ("hard_hardgate_n48", 1, 60, 3, 48, 16, 1, 1, 1),
]


def make_keyless_case(name, B, T, H, N, DV, G, hard, hard_gate, seed):
    """ref_scan_v in float64 (gqa25/slotkern_v.py:242-261), gradients by autograd; inputs as in its self-test (:275-279)."""
    import slotkern_v as SV
    gen = torch.Generator().manual_seed(seed)
    v = torch.randn(B, T, H, DV, generator=gen).double()
    wa = (1.5 * torch.randn(B, T, H, N, generator=gen)).double()
    gate = torch.sigmoid(torch.randn(B, T, H, generator=gen)).double()
    fr = torch.tensor([3.0], dtype=torch.float64)
    leaves = [x.clone().requires_grad_() for x in (v, wa, gate, fr)]
    buf = SV.ref_scan_v(*leaves, N, G=G, hard=bool(hard), hard_gate=bool(hard_gate))
    w = torch.randn(buf.shape, generator=gen).double()
    (buf * w).sum().backward()
    np.savez_compressed(os.path.join(HERE, "keyless_%s.npz" % name), v=v.float().numpy(), wa=wa.float().numpy(),
                        gate=gate.float().numpy(), fr=fr.float().numpy(), buf=buf.detach().numpy(), w=w.float().numpy(),
                        dv=leaves[0].grad.numpy(), dwa=leaves[1].grad.numpy(), dgate=leaves[2].grad.numpy(),
                        dfr=leaves[3].grad.numpy(), meta=np.array([B, T, H, N, DV, G, hard, hard_gate], np.int64))
    print("keyless_%s.npz  buf %s" % (name, tuple(buf.shape)))


if __name__ == "__main__":
    torch.set_num_threads(8)
    if "--keyless-only" in sys.argv:
        for i, case in enumerate(KEYLESS_CASES):
            make_keyless_case(*case, seed=400 + i)
        sys.exit(0)
    for i, case in enumerate(SCAN_CASES):
        make_scan_case(*case, seed=100 + i)
    for i, case in enumerate(KEYLESS_CASES):
        make_keyless_case(*case, seed=400 + i)
    make_read_case()
    make_quant_case()
