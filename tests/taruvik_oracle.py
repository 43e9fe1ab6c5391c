"""Slow fp32 restatement of the Taruvik design, one function per mechanism, on plain torch CPU tensors.  It shares no code with
the product path: whole sequences, no cache, every key of every head materialised.

A model is (cfg, W): cfg the dict of config.json, W a dict of checkpoint-named fp32 tensors.
"""
import math
from typing import Dict, List, Optional

import torch

Tensors = Dict[str, torch.Tensor]


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def yarn_frequencies(rot: dict) -> (torch.Tensor, float):
    """Per-pair angular frequencies (float64) and the magnitude both cos and sin are multiplied by."""
    n, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / n) for i in range(n // 2)], dtype=torch.float64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns: float) -> float:
        return n * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), n - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(n // 2)], dtype=torch.float64)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(v: torch.Tensor, pos: torch.Tensor, rot: dict) -> torch.Tensor:
    """v [T, ..., n >= dims]: rotates the pairs (2i, 2i+1) of the first rot.dims entries by pos * f_i; the rest pass."""
    n = int(rot["dims"])
    f, mag = yarn_frequencies(rot)
    ang = pos.double()[:, None] * f[None, :]                      # [T, n/2]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [n // 2]
    c, s = (torch.cos(ang) * mag).float().view(shape), (torch.sin(ang) * mag).float().view(shape)
    a, b = v[..., 0:n:2], v[..., 1:n:2]
    out = v.clone()
    out[..., 0:n:2] = a * c - b * s
    out[..., 1:n:2] = b * c + a * s
    return out


def latent_attention(h: torch.Tensor, W: Tensors, p: str, m: dict, eps: float, pos: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h [T, width] of ONE sequence at positions pos (default 0..T-1) -> mixer output [T, width]."""
    T = h.shape[0]
    pos = torch.arange(T) if pos is None else pos
    H, dn, dr, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = rms_norm(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).view(T, H, dn + dr)
    kv = h @ W[p + "dkv"].T
    c = rms_norm(kv[:, :r], W[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(kv[:, r:], pos, m["rot"])                 # [T, dr], one for all heads
    q_rot = rotate_pairs(q[..., dn:], pos, m["rot"])               # [T, H, dr]
    k_n = (c @ W[p + "uk"].T).view(T, H, dn)
    val = (c @ W[p + "uv"].T).view(T, H, dv)
    s = torch.einsum("thd,shd->hts", q[..., :dn], k_n) + torch.einsum("thd,sd->hts", q_rot, k_rot)
    s = s * float(m["scale"])
    seen = pos[None, :] <= pos[:, None]
    s = s.masked_fill(~seen[None], float("-inf"))
    o = torch.einsum("hts,shd->thd", torch.softmax(s, -1), val)
    gate = torch.sigmoid(h @ W[p + "g"].T)                         # [T, H]
    return (o * gate[..., None]).reshape(T, H * dv) @ W[p + "o"].T


def route(h: torch.Tensor, W: Tensors, p: str, r: dict) -> torch.Tensor:
    """Dense routing weights [T, experts + identity]: the score of every chosen expert, 0 elsewhere."""
    n = int(r["experts"]) + int(r.get("identity", 0))
    s = torch.softmax(h @ W[p + "router"].T, -1)
    choice = s + W[p + "correction"]
    g = r.get("groups")
    if g:
        cnt, keep = int(g["count"]), int(g["keep"])
        best = choice.view(-1, cnt, n // cnt).max(-1).values
        kept = torch.zeros_like(best, dtype=torch.bool).scatter_(1, best.topk(keep, -1).indices, True)
        choice = choice.masked_fill(~kept.repeat_interleave(n // cnt, 1), float("-inf"))
    idx = choice.topk(int(r["top"]), -1).indices
    return torch.zeros_like(s).scatter_(1, idx, s.gather(1, idx))


def moe(h: torch.Tensor, W: Tensors, p: str, a: dict) -> torch.Tensor:
    r = a["router"]
    E = int(r["experts"])
    wts = route(h, W, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.nonzero(wts[t]).flatten().tolist():
            if e >= E:
                y = h[t]
            else:
                q = f"{p}e{e}."
                g = W[q + "gate"] @ h[t]
                y = W[q + "down"] @ (g * torch.sigmoid(g) * (W[q + "up"] @ h[t]))
            out[t] += wts[t, e] * y
    return out


def layer_schedule(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    a, b, k = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n))


def forward(cfg: dict, W: Tensors, tokens: List[int], taps: Optional[list] = None) -> torch.Tensor:
    """fp32 logits [T, vocab] of one whole sequence; `taps` collects the residual stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x0 = W["embed"][torch.tensor(tokens)]
    x = x0.clone()
    lp = cfg.get("loop")
    runs = layer_schedule(cfg)
    seen_first = False
    for i in runs:
        if lp and i == int(lp["start"]):
            if seen_first:
                x = x + x0
            seen_first = True
        L, p = cfg["layers"][i], f"l{i}."
        assert L["type"] == "latent_attention"

        def ln(name: str, v: torch.Tensor) -> torch.Tensor:
            return layer_norm(v, W[p + name], W[p + name + ".b"], eps)

        x = x + ln("norm1b", latent_attention(ln("norm1", x), W, p + "mix.", L["mixer"], eps))
        if L.get("mlp") is not None:
            assert L["mlp"]["kind"] == "moe"
            x = x + ln("norm2b", moe(ln("norm2", x), W, p + "mlp.", L["mlp"]))
        if taps is not None:
            taps.append(x.clone())
    return layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
