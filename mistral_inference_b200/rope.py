"""RoPE table (mirror of mistral_inference/rope.py:6-10).

The table is built on the CPU in fp32 exactly as the reference does (transformer.py:108-120 builds it on
the default device, then moves it) and uploaded, so the kernels multiply by the very same cos/sin bits
instead of calling sincosf on the device.  The rotation itself
(rope.py:13-23) is the epilogue of the fused QKV kernel (csrc/epilogue.cuh, EPI_QKV_ROPE).
"""
import torch


def precompute_freqs_cis(dim: int, end: int, theta: float) -> torch.Tensor:
    """complex64 [end, dim/2]: polar(1, t * theta^(-2i/dim))."""
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2)[: (dim // 2)].float() / dim))
    t = torch.arange(end, device=freqs.device)
    freqs = torch.outer(t, freqs).float()
    return torch.polar(torch.ones_like(freqs), freqs)


def scaled_frequencies(dims: int, base: float, scaling=None):
    """(float64 [dims/2] angular frequencies per position step, magnitude of cos and sin) of a rotation over `dims` entries with
    optional YaRN-style frequency scaling (scaling: factor, original context, and the numbers of turns `fast` / `slow` over that
    context between which the pairs go from unscaled to divided by `factor`):
        f_i = base^(-2i/dims);  turn_dim(t) = dims ln(original / (2 pi t)) / (2 ln base)
        lo = max(floor(turn_dim(fast)), 0), hi = min(ceil(turn_dim(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        f'_i = f_i / factor * ramp_i + f_i (1 - ramp_i);  magnitude = 0.1 ln(factor) + 1
    Evaluated on the host in double precision; the kernels multiply positions by these in double as well."""
    import math
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling.factor), float(scaling.original)

    def turn_dim(turns: float) -> float:
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling.fast))), 0)
    hi = min(math.ceil(turn_dim(float(scaling.slow))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0
