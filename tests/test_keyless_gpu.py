"""GPU parity of the keyless scan (slot_scan_v) against the reference's golden vectors and the float64 oracle.
Tolerances: the reference's own self-test accepts buf 2e-4 and gradients 2e-3 relative to the tensor's max
(gqa25/slotkern_v.py:270); here float32 mode is held to rtol = atol = 1e-5 on the buffer and 1e-4 on the gradients."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.scan_cases import allclose_report, rel_to_max

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DEV = "cuda"
KEYLESS = sorted(glob.glob(os.path.join(GOLDEN, "keyless_*.npz")))


def run(v, wa, gate, fr, N, G, hard, hard_gate, w, dtype=torch.float32, buf_dtype=torch.float32):
    import slotscan_b200 as S
    leaves = [torch.as_tensor(np.asarray(x, np.float32)).to(DEV, dt).requires_grad_()
              for x, dt in ((v, dtype), (wa, torch.float32), (gate, torch.float32), (fr, torch.float32))]
    buf = S.slot_scan_v(*leaves, N, G=G, hard=hard, hard_gate=hard_gate, buf_dtype=buf_dtype)
    (buf.float() * torch.as_tensor(np.asarray(w, np.float32)).to(DEV)).sum().backward()
    return buf.detach().float().cpu().numpy(), [t.grad.float().cpu().numpy() for t in leaves]


@pytest.mark.parametrize("path", KEYLESS, ids=[os.path.basename(p)[8:-4] for p in KEYLESS])
def test_keyless_golden_reference_vectors(path):
    z = np.load(path)
    B, T, H, N, DV, G, hard, hard_gate = (int(x) for x in z["meta"])
    buf, grads = run(z["v"], z["wa"], z["gate"], z["fr"], N, G, bool(hard), bool(hard_gate), z["w"])
    okc, worst = allclose_report(buf, z["buf"], 1e-5, 1e-5)
    assert okc, worst
    assert np.abs(buf[:, 0]).max() == 0                                    # snapshot 0 is the empty memory
    for g, n in zip(grads, ("dv", "dwa", "dgate", "dfr")):
        assert rel_to_max(g.reshape(z[n].shape), z[n]) < 1e-4, n


@pytest.mark.parametrize("case", [(2, 100, 3, 48, 16, 1, True, True), (1, 300, 2, 48, 16, 4, True, False),
                                  (3, 63, 4, 16, 16, 1, False, False), (1, 37, 2, 200, 40, 8, False, True)],
                         ids=["N48_hard_hardgate", "T300_G4_hard", "N16_soft", "N200_D40_TmodG"])
def test_keyless_vs_float64_oracle(case):
    """The shapes of the reference's self-test (gqa25/slotkern_v.py:283-289) and one wide one, seeded as there."""
    B, T, H, N, DV, G, hard, hard_gate = case
    gen = torch.Generator().manual_seed(1234)
    v = torch.randn(B, T, H, DV, generator=gen)
    wa = 1.5 * torch.randn(B, T, H, N, generator=gen)
    gate = torch.sigmoid(torch.randn(B, T, H, generator=gen))
    fr = torch.tensor([3.0])
    ref = O.scan_v_fwd(v, wa, gate, fr, N, G=G, hard=hard, hard_gate=hard_gate)
    w = torch.randn(ref["buf"].shape, generator=gen).numpy()
    gr = O.scan_v_bwd(v, wa, gate, fr, N, w, G=G, hard=hard, hard_gate=hard_gate)
    buf, grads = run(v.numpy(), wa.numpy(), gate.numpy(), fr.numpy(), N, G, hard, hard_gate, w)
    okc, worst = allclose_report(buf, ref["buf"], 1e-5, 1e-5)
    assert okc, worst
    for g, n in zip(grads, ("dv", "dwa", "dgate", "dfr")):
        assert rel_to_max(g.reshape(gr[n].shape), gr[n]) < 1e-4, n


def test_keyless_contract():
    """bf16 values and buffer, bitwise repeatability (the reference checks it too, slotkern_v.py:298-305), no CPU path."""
    import slotscan_b200 as S
    import slotkern_v
    assert slotkern_v.slot_scan_v is S.slot_scan_v
    gen = torch.Generator().manual_seed(5)
    B, T, H, DV, N = 2, 90, 4, 16, 48
    v, wa = torch.randn(B, T, H, DV, generator=gen).to(DEV), torch.randn(B, T, H, N, generator=gen).to(DEV)
    gate, fr = torch.rand(B, T, H, generator=gen).to(DEV), torch.tensor([2.0], device=DEV)

    def once():
        ins = [x.clone().requires_grad_() for x in (v, wa, gate, fr)]
        b = S.slot_scan_v(*ins, N, C=32, hard=True, hard_gate=True)
        b.sum().backward()
        return [b] + [t.grad for t in ins]
    r1, r2 = once(), once()
    assert all(torch.equal(a, b) for a, b in zip(r1, r2))
    b16 = S.slot_scan_v(v.to(torch.bfloat16), wa, gate, fr, N, G=4, buf_dtype=torch.bfloat16, hard=True)
    b32 = S.slot_scan_v(v.to(torch.bfloat16).float(), wa, gate, fr, N, G=4, hard=True)
    assert b16.dtype == torch.bfloat16 and b16.shape == (B, 23, H, N, DV) and torch.equal(b16, b32.to(torch.bfloat16))
    with pytest.raises(RuntimeError):
        S.slot_scan_v(v.cpu(), wa.cpu(), gate.cpu(), fr.cpu(), N)
