"""Plain, slow fp32 statement of the Fesenex design, one function per mechanism, on the CPU.

Nothing here is shared with the product path (`mistral_inference_b200`): the tests compare the CUDA
kernels and the cache / scheduler against these loops.  Weights arrive as a dict name -> tensor with the
checkpoint's names (`embed`, `l<i>.norm1`, `l<i>.mix.q`, ..., `final.norm`, `head`); `cfg` is the parsed
config.json.  Everything is computed in float64-free, straightforward float32 torch.
"""
import math
from typing import Dict, List, Optional

import torch

GELU_C = math.sqrt(2.0 / math.pi)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * w


def rel_bucket(n: int, rows: int, far: float) -> int:
    """Row of the distance table for distance n >= 0: identity below rows/2, then logarithmic up to `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def q_temperature(pos: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((pos + 1) // every + 1)


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                    v_first: Optional[torch.Tensor], is_first_vmix: bool):
    """h [n, width] of ONE sequence from position 0.  Returns (out [n, width], values as cached [n, G*vdim])."""
    n = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(n, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(n, G, d)
    v = h @ w[p + "v"].T + w[p + "v.b"]
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    if m.get("q_temp"):
        t = torch.tensor([q_temperature(i, m["q_temp"]["coef"], m["q_temp"]["every"]) for i in range(n)])
        q = q * t[:, None, None]
    if m.get("v_mix") and not is_first_vmix:
        lam = w[p + "vmix"].float()
        v = (1.0 - lam) * v + lam * v_first
    vv = v.view(n, G, e)
    rel = w[p + "rel"]
    rows = rel.shape[0]
    out = torch.zeros(n, H, e)
    for i in range(n):
        for hh in range(H):
            g = hh // (H // G)
            s = torch.empty(i + 1)
            for j in range(i + 1):
                s[j] = (q[i, hh] @ k[j, g]) * m["scale"] + rel[rel_bucket(i - j, rows, m["bias_max"]), hh]
            a = torch.softmax(s, 0)
            out[i, hh] = a @ vv[: i + 1, g]
    return out.reshape(n, H * e) @ w[p + "o"].T, v


def lightning_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                    state: Optional[torch.Tensor] = None):
    """Decayed linear attention, token by token.  state [H, d, e] (zeros when None).  Returns (out, state)."""
    n = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(h @ w[p + "q"].T).view(n, H, d)
    k = silu(h @ w[p + "k"].T).view(n, H, d)
    v = silu(h @ w[p + "v"].T).view(n, H, e)
    S = torch.zeros(H, d, e) if state is None else state.clone()
    o = torch.zeros(n, H, e)
    for t in range(n):
        for hh in range(H):
            S[hh] = m["decay"][hh] * S[hh] + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    y = norm(o.reshape(n, H * e), w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T, S


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    lim = f["limit"]
    g = torch.clamp(h @ w[p + "gate"].T, max=lim)
    u = torch.clamp(h @ w[p + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one whole sequence."""
    w = {k: (v.float() if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        hn = norm(x, w[p + "norm1"], eps)
        if L["type"] == "attention":
            first = bool(L["mixer"].get("v_mix")) and v_first is None
            y, v = attention_mixer(hn, w, p + "mix.", L["mixer"], eps, v_first, first)
            if first:
                v_first = v
        elif L["type"] == "lightning":
            y, _ = lightning_mixer(hn, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + y
        if L.get("mlp") is not None:
            assert L["mlp"]["kind"] == "dense"
            x = x + dense_ff(norm(x, w[p + "norm2"], eps), w, p + "mlp.", L["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm(x, w["final.norm"], eps) @ w["head"].T
