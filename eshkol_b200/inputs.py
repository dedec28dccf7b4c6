"""Seeded synthetic operands.

The uniform stream is the reference runtime's 48-bit LCG (lib/core/prng.cpp:45-58,
76-80: state0 = (seed << 16) | 0x330E, state' = state * 0x5DEECE66D + 0xB mod 2^48,
u = state / 2^48), evaluated with a skip-ahead so that numpy (host) and torch
(device) produce the same states.  The distributions on top of it are this
project's own definitions of the benchmark configurations:

  uniform       2u - 1                                   (one draw per element)
  wide          (2u - 1) * 2^k, k = floor(41 u') - 20    (two draws per element)
  normal        Box-Muller on consecutive draws, scaled  (two draws per pair)
  full53        +-m/2^53, m a 53-bit integer from two draws  (parity only)
"""
from __future__ import annotations

import math

import numpy as np

_A = 0x5DEECE66D
_C = 0xB
_MASK = (1 << 48) - 1


def seed_state(seed: int) -> int:
    return ((seed << 16) | 0x330E) & _MASK


def _skip_tables(n: int, xp):
    """A[i], Cc[i] with state_{i+1..n} = A[i]*state0 + Cc[i] (mod 2^48), by doubling."""
    if xp is np:
        A = np.empty(n, dtype=np.uint64)
        Cc = np.empty(n, dtype=np.uint64)
        mask = np.uint64(_MASK)
    else:
        import torch
        A = torch.empty(n, dtype=torch.int64, device=xp_device(xp))
        Cc = torch.empty(n, dtype=torch.int64, device=xp_device(xp))
        mask = _MASK
    A[0] = _A
    Cc[0] = _C
    am, cm, m = _A, _C, 1  # a^m, c_m for the current prefix length m
    while m < n:
        take = min(m, n - m)
        if xp is np:
            with np.errstate(over="ignore"):
                A[m:m + take] = (A[:take] * np.uint64(am)) & mask
                Cc[m:m + take] = (Cc[:take] * np.uint64(am) + np.uint64(cm)) & mask
        else:
            am_s = am if am < (1 << 63) else am - (1 << 64)
            A[m:m + take] = (A[:take] * am_s) & mask
            Cc[m:m + take] = (Cc[:take] * am_s + cm) & mask
        # a^(2m), c_(2m) = a^m * c_m + c_m
        cm = (am * cm + cm) & _MASK
        am = (am * am) & _MASK
        m += take
    return A, Cc


class _TorchXP:
    def __init__(self, device):
        self.device = device


def xp_device(xp):
    return xp.device


def _advance(state: int, steps: int) -> int:
    """state after `steps` LCG steps, by square-and-multiply on the affine map"""
    am, cm = _A, _C
    acc_a, acc_c = 1, 0
    while steps:
        if steps & 1:
            acc_a, acc_c = (acc_a * am) & _MASK, (acc_c * am + cm) & _MASK
        cm = (am * cm + cm) & _MASK
        am = (am * am) & _MASK
        steps >>= 1
    return (acc_a * state + acc_c) & _MASK


def lcg_states(seed: int, n: int, device=None, start: int = 0):
    """states start+1..start+n of the stream seeded with `seed` (numpy uint64, or torch
    int64 on `device`)."""
    s0 = _advance(seed_state(seed), start)
    if device is None:
        A, Cc = _skip_tables(n, np)
        with np.errstate(over="ignore"):
            return (A * np.uint64(s0) + Cc) & np.uint64(_MASK)
    xp = _TorchXP(device)
    A, Cc = _skip_tables(n, xp)
    return (A * s0 + Cc) & _MASK


def _to_unit(states, device):
    if device is None:
        return states.astype(np.float64) * (1.0 / float(1 << 48))
    import torch
    return states.to(torch.float64) * (1.0 / float(1 << 48))


def uniform(seed: int, shape, device=None, start: int = 0):
    """entries 2u - 1 in [-1, 1), row-major fill order; `start` skips that many elements
    of the stream (a row shard of a larger matrix)"""
    n = int(np.prod(shape))
    u = _to_unit(lcg_states(seed, n, device, start), device)
    return (2.0 * u - 1.0).reshape(*shape)


def wide(seed: int, shape, device=None, span: int = 41, lo: int = -20):
    """(2u - 1) * 2^k with k uniform in [lo, lo + span): wide exponent range"""
    n = int(np.prod(shape))
    u = _to_unit(lcg_states(seed, 2 * n, device), device)
    base = 2.0 * u[0::2] - 1.0
    if device is None:
        k = np.floor(span * u[1::2]).astype(np.int64) + lo
        return np.ldexp(base, k).reshape(*shape)
    import torch
    k = torch.floor(span * u[1::2]).to(torch.int32) + lo
    return torch.ldexp(base, k).reshape(*shape)


def normal(seed: int, shape, device=None, scale: float = 1.0):
    """Box-Muller on consecutive draws (u1 shifted into (0, 1])"""
    n = int(np.prod(shape))
    npair = (n + 1) // 2
    st = lcg_states(seed, 2 * npair, device)
    if device is None:
        u1 = (st[0::2].astype(np.float64) + 1.0) * (1.0 / float(1 << 48))
        u2 = st[1::2].astype(np.float64) * (1.0 / float(1 << 48))
        r = np.sqrt(-2.0 * np.log(u1))
        z = np.empty(2 * npair, dtype=np.float64)
        z[0::2] = r * np.cos(2.0 * math.pi * u2)
        z[1::2] = r * np.sin(2.0 * math.pi * u2)
        return (scale * z[:n]).reshape(*shape)
    import torch
    u1 = (st[0::2].to(torch.float64) + 1.0) * (1.0 / float(1 << 48))
    u2 = st[1::2].to(torch.float64) * (1.0 / float(1 << 48))
    r = torch.sqrt(-2.0 * torch.log(u1))
    z = torch.empty(2 * npair, dtype=torch.float64, device=device)
    z[0::2] = r * torch.cos(2.0 * math.pi * u2)
    z[1::2] = r * torch.sin(2.0 * math.pi * u2)
    return (scale * z[:n]).reshape(*shape)


def full53(seed: int, shape, device=None):
    """+-m / 2^53 with m a 53-bit integer built from the high bits of two draws (32 of
    the first, 21 of the second; the sign is bit 20 of the second).  The low bits of
    the LCG states have short periods and are not used.  Every mantissa bit down to
    2^-53 varies, so the scaled operands take odd as well as even integer values."""
    n = int(np.prod(shape))
    st = lcg_states(seed, 2 * n, device)
    if device is None:
        m = ((st[0::2] >> np.uint64(16)) << np.uint64(21)) | (st[1::2] >> np.uint64(27))
        sign = 1.0 - 2.0 * ((st[1::2] >> np.uint64(20)) & np.uint64(1)).astype(np.float64)
        return (sign * (m.astype(np.float64) * (1.0 / float(1 << 53)))).reshape(*shape)
    import torch
    m = ((st[0::2] >> 16) << 21) | (st[1::2] >> 27)
    sign = 1.0 - 2.0 * ((st[1::2] >> 20) & 1).to(torch.float64)
    return (sign * (m.to(torch.float64) * (1.0 / float(1 << 53)))).reshape(*shape)
