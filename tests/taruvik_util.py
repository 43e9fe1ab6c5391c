"""Small random Taruvik models for the tests: configurations, weights with the checkpoint's names, folders on disk."""
import json
import math
from pathlib import Path
from typing import Dict, Optional

import torch


def mixer_cfg(**over) -> dict:
    m = {"heads": 3, "dim": 12, "rot_dim": 8, "vdim": 20, "q_rank": 24, "kv_rank": 40, "scale": 0.3,
         "rot": {"base": 1000.0, "dims": 8, "scaling": {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 1.0}}}
    m.update(over)
    return m


def moe_cfg(ff=24, experts=6, top=3, identity=2, count=4, keep=2) -> dict:
    r = {"experts": experts, "top": top, "identity": identity}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def make_config(width=40, vocab=50, layers=None, loop=None, eps=1e-4) -> dict:
    """layers: list of (mixer dict, mlp dict or None)."""
    cfg = {"architecture": "Taruvik", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [{"type": "latent_attention", "mixer": m, "mlp": f} for m, f in layers]}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def make_weights(cfg: dict, seed: int = 0, dtype=torch.float32, router_gain: float = 4.0, correction: float = 0.15) -> Dict[str, torch.Tensor]:
    """The default correction is comparable to the scores: it changes choices and can make choice scores negative."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s / math.sqrt(i)).to(dtype)

    def vec(n, mean=0.0, s=0.3):
        return (mean + s * torch.randn(n, generator=g)).to(dtype)

    w = {"embed": (torch.randn(cfg["vocab"], W, generator=g)).to(dtype), "head": mat(cfg["vocab"], W), "final.norm": vec(W, 1.0), "final.norm.b": vec(W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L["mlp"] else ()):
            w[p + n], w[p + n + ".b"] = vec(W, 1.0), vec(W)
        H, dn, dr, dv, rq, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
        w[p + "mix.dq"], w[p + "mix.dq.norm"], w[p + "mix.uq"] = mat(rq, W), vec(rq, 1.0), mat(H * (dn + dr), rq, 2.0)
        w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(rk + dr, W, 2.0), vec(rk, 1.0)
        w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * dn, rk, 2.0), mat(H * dv, rk)
        w[p + "mix.g"], w[p + "mix.o"] = mat(H, W, 3.0), mat(W, H * dv)
        if L["mlp"]:
            r, ff = L["mlp"]["router"], L["mlp"]["expert"]["ff"]
            n = r["experts"] + r.get("identity", 0)
            w[p + "mlp.router"] = mat(n, W, router_gain)
            w[p + "mlp.correction"] = vec(n, 0.0, correction)  # comparable to the scores: changes choices, can make choice scores negative
            for e in range(r["experts"]):
                w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = mat(ff, W, 2.0), mat(ff, W, 2.0), mat(W, ff, 2.0)
    return w


def write_folder(path: Path, cfg: dict, weights: Dict[str, torch.Tensor]) -> Path:
    from safetensors.torch import save_file

    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(path / "model.safetensors"))
    return path


def f32(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.float() for k, v in weights.items()}
