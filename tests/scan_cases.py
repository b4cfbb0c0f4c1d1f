"""Seeded input generators and comparison helpers shared by the GPU parity tests, smoke() and bench.py's checks.

Distributions:
  bench      the benchmark configuration's: unit keys, 0.5 randn values, sigmoid gates, fr = 0.1 randn per token,
             independent unit write query, temp 16
  clustered  gqa25/test_frtok.py:13-36: keys drawn around 6 centres so occupied rows compete with the free row,
             fr / temp in [0.2, 1.5]
  gates01    kvu/test_cuda.py:21-28: randn keys, gates forced to exact 0 (15 %) and exact 1 (8 %), fr in [0, 2);
             "gates01:S" draws fr in [0, S) instead: S = 3 uses ~55 of 192 rows, S = 4 ~110 (the row counts at which
             the kernels switch variants), S = 6 all of them
  fill       every row gets used: strong free-row preference until the memory is full, then pure matching
All tensors are drawn on the CPU in float32 from one torch.Generator, in a fixed order.
"""
import numpy as np
import torch


def make_inputs(dist, B, T, H, DK, DV, seed, frtok=True, sepq=True):
    gen = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=gen)
    u = lambda *s: torch.rand(*s, generator=gen)
    unit = lambda x: x / x.norm(dim=-1, keepdim=True)
    temp = 16.0
    if dist == "bench":
        k, v = unit(r(B, T, H, DK)), 0.5 * r(B, T, H, DV)
        g = torch.sigmoid(r(B, T, H))
        fr = 0.1 * r(B, T, H) if frtok else torch.tensor([0.05])
        q = unit(r(B, T, H, DK)) if sepq else None
    elif dist == "clustered":
        cen = r(B, 6, H, DK)
        idx = torch.randint(0, 6, (B, T), generator=gen)
        k = torch.gather(cen, 1, idx[:, :, None, None].expand(B, T, H, DK)) + 0.3 * r(B, T, H, DK)
        q = k + 0.2 * r(B, T, H, DK) if sepq else None
        v, g = r(B, T, H, DV), u(B, T, H)
        fr = temp * (0.2 + 1.3 * u(B, T, H)) if frtok else torch.tensor([9.0])
    elif dist.startswith("gates01"):
        frs = float(dist.split(":")[1]) if ":" in dist else 2.0
        k, q, v = r(B, T, H, DK), (r(B, T, H, DK) if sepq else None), r(B, T, H, DV)
        g, m = u(B, T, H), u(B, T, H)
        g = torch.where(m < 0.15, torch.zeros_like(g), torch.where(m > 0.92, torch.ones_like(g), g))
        fr = frs * u(B, T, H) if frtok else torch.tensor([0.75 * frs])
    elif dist == "fill":
        # every row gets used: a strong free-row preference until the memory is full, then pure matching
        k, v = unit(r(B, T, H, DK)), 0.5 * r(B, T, H, DV)
        g = torch.sigmoid(r(B, T, H) + 1.0)
        fr = 4.0 + 0.5 * r(B, T, H) if frtok else torch.tensor([4.0])
        q = unit(k + 0.5 * unit(r(B, T, H, DK))) if sepq else None
    else:
        raise ValueError(dist)
    return dict(k=k, q=q, v=v, gate=g, fr=fr, temp=temp)


def rel_to_max(a, b):
    """max |a-b| / max |b|: the reference's gradient criterion (kvu/test_cuda.py:50)."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def allclose_report(a, b, rtol, atol):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    err = np.abs(a - b) - (atol + rtol * np.abs(b))
    return bool((err <= 0).all()), float(err.max())


def bf16_round(x):
    """x rounded to bfloat16 (round to nearest even) and back, as float64."""
    return torch.as_tensor(np.asarray(x, np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


def bf16_band_report(out, ref, scale=1.0):
    """A bf16-typed result against the oracle.  bf16 keeps 8 significant bits (unit round-off 2^-8 = 3.9e-3), so a
    stored number cannot sit within rtol 2e-3 of the exact one; what can be asked is that it IS the oracle's value in
    that storage format.  Returns (inside, worst, share):
      inside  every element within one bf16 ulp of the bf16-rounded oracle value, plus atol 2e-3 of `scale`
      worst   the largest excess over that band
      share   the fraction of elements that are NOT bit-identical to the bf16-rounded oracle value.  float32
              round-off tips a value across a rounding boundary only rarely, so a kernel that is one ulp off
              everywhere passes `inside` but fails a bound on `share`."""
    r = bf16_round(ref)
    o = np.asarray(out, np.float64)
    err = np.abs(o - r) - (np.abs(r) * 2.0 ** -7 + 2e-3 * scale)
    return bool((err <= 0).all()), float(err.max()), float((o != r).mean())


def address_report(addr, ref_addr, margin, tol=1e-4):
    """Addresses must agree wherever the oracle's top-1 / top-2 margin exceeds `tol`.  A flip at a near-tie changes
    everything after it in that (sequence, head), so those sequences are reported and left out of value checks.
    Returns (ok, n_flips_total, n_bad (flips with margin > tol), keep mask over (B,H))."""
    addr, ref_addr, margin = (np.asarray(x) for x in (addr, ref_addr, margin))
    B, T, H = addr.shape
    diff = addr != ref_addr
    keep = np.ones((B, H), bool)
    n_bad = 0
    for b in range(B):
        for h in range(H):
            d = np.nonzero(diff[b, :, h])[0]
            if d.size:
                keep[b, h] = False
                if margin[b, d[0], h] > tol:          # only the FIRST divergence is attributable to rounding
                    n_bad += 1
    return n_bad == 0, int((~keep).sum()), n_bad, keep
