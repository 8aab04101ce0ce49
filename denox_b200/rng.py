"""Seeded synthetic tensors, independent of torch / numpy generator versions.

splitmix64 counter-based stream -> uniform [0, 1) with 53 bits -> (Box-Muller)
normal.  Values are produced in float64, rounded once to float32 and once more
(round to nearest even) to binary16 by numpy.
"""
import numpy as np

_MASK = np.uint64(0xFFFFFFFFFFFFFFFF)


def splitmix64(seed: int, n: int) -> np.ndarray:
    """n successive outputs of splitmix64 started at `seed` (vectorised: the state is a counter)."""
    with np.errstate(over="ignore"):
        i = np.arange(1, n + 1, dtype=np.uint64)
        z = (np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + i * np.uint64(0x9E3779B97F4A7C15)) & _MASK
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _MASK
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _MASK
        return z ^ (z >> np.uint64(31))


def uniform(seed: int, n: int, lo: float = 0.0, hi: float = 1.0) -> np.ndarray:
    u = (splitmix64(seed, n) >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)
    return lo + (hi - lo) * u


def normal(seed: int, n: int, std: float = 1.0) -> np.ndarray:
    m = (n + 1) // 2
    u = uniform(seed, 2 * m)
    u1 = 1.0 - u[:m]  # (0, 1]
    u2 = u[m:]
    r = np.sqrt(-2.0 * np.log(u1))
    z = np.concatenate([r * np.cos(2.0 * np.pi * u2), r * np.sin(2.0 * np.pi * u2)])[:n]
    return z * std


def to_f16(x: np.ndarray) -> np.ndarray:
    return x.astype(np.float32).astype(np.float16)


def he_normal_weights(seed: int, c_out: int, c_in: int) -> np.ndarray:
    """[c_out][c_in][3][3] binary16, N(0, 2 / (9 c_in))."""
    std = float(np.sqrt(2.0 / (9.0 * c_in)))
    return to_f16(normal(seed, c_out * c_in * 9, std)).reshape(c_out, c_in, 3, 3)


def uniform_torch(seed: int, n: int, lo: float = 0.0, hi: float = 1.0, device="cuda"):
    """`uniform` evaluated with torch on `device`: the same float64 values, bit for bit (64-bit integer
    arithmetic wraps the same way; unsigned shifts are emulated with masks).  Returns a float64 tensor."""
    import torch
    i64 = torch.int64

    def c(v):  # 64-bit constant as a signed value
        v &= 0xFFFFFFFFFFFFFFFF
        return v - (1 << 64) if v >= (1 << 63) else v

    def lsr(z, k):  # logical shift right
        return (z >> k) & ((1 << (64 - k)) - 1)

    i = torch.arange(1, n + 1, dtype=i64, device=device)
    z = i * c(0x9E3779B97F4A7C15) + c(seed)
    z = (z ^ lsr(z, 30)) * c(0xBF58476D1CE4E5B9)
    z = (z ^ lsr(z, 27)) * c(0x94D049BB133111EB)
    z = z ^ lsr(z, 31)
    u = lsr(z, 11).to(torch.float64) * (1.0 / 9007199254740992.0)
    return lo + (hi - lo) * u
