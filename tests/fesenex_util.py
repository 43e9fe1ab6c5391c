"""Small random Fesenex models for the tests: configurations, weights with the checkpoint's names, folders on disk."""
import json
import math
from pathlib import Path
from typing import Dict, List, Optional

import torch


def make_config(width=48, vocab=64, layers=None, eps=1e-3, emb_scale=None) -> dict:
    """layers: list of (type, mixer overrides[, mlp overrides or None])."""
    out = []
    for item in layers:
        kind, mix = item[0], dict(item[1])
        mlp = item[2] if len(item) > 2 else {}
        if kind == "attention":
            m = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.2, "bias_max": 40, "v_mix": False,
                 "q_temp": {"coef": 0.4, "every": 5}, "_rel_rows": 8}
            m.update(mix)
            if m.get("q_temp") is None:
                m.pop("q_temp")
        else:
            m = {"heads": 2, "dim": 16, "vdim": 8}
            m.update(mix)
            m.setdefault("decay", [math.exp(-1.0 / (2 + 3 * h)) for h in range(m["heads"])])
        out.append({"type": kind, "mixer": m, "mlp": None if mlp is None else {"kind": "dense", "ff": 40, "limit": 1.5, **mlp}})
    return {"architecture": "Fesenex", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale or math.sqrt(width)},
            "norm": {"eps": eps}, "layers": out}


def make_weights(cfg: dict, seed: int = 0, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s / math.sqrt(i)).to(dtype)

    def vec(n, mean=0.0, s=0.5):
        return (mean + s * torch.randn(n, generator=g)).to(dtype)

    w = {"embed": (torch.randn(cfg["vocab"], W, generator=g) / math.sqrt(W)).to(dtype), "final.norm": vec(W, 1.0, 0.2), "head": mat(cfg["vocab"], W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"] = vec(W, 1.0, 0.2)
        if L["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.q.b"] = mat(H * d, W, 2.0), vec(H * d)
            w[p + "mix.k"], w[p + "mix.k.b"] = mat(G * d, W, 2.0), vec(G * d)
            w[p + "mix.v"], w[p + "mix.v.b"] = mat(G * e, W), vec(G * e)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = vec(d, 1.0, 0.3), vec(d, 1.0, 0.3)
            w[p + "mix.rel"] = (torch.randn(m.get("_rel_rows", 8), H, generator=g) * 1.5).to(dtype)
            w[p + "mix.vmix"] = torch.tensor(0.3 + 0.1 * i).to(dtype)
            w[p + "mix.o"] = mat(W, H * e)
        else:
            H, d, e = m["heads"], m["dim"], m["vdim"]
            for n, o in (("q", H * d), ("k", H * d), ("v", H * e), ("g", H * e)):
                w[p + "mix." + n] = mat(o, W, 2.0)
            w[p + "mix.norm"] = vec(H * e, 1.0, 0.3)
            w[p + "mix.o"] = mat(W, H * e)
        if L["mlp"] is not None:
            ff = L["mlp"]["ff"]
            w[p + "norm2"] = vec(W, 1.0, 0.2)
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, W, 3.0), mat(ff, W, 3.0), mat(W, ff)
    return w


def clean_config(cfg: dict) -> dict:
    """Without the keys that only steer the test's weight maker."""
    c = json.loads(json.dumps(cfg))
    for L in c["layers"]:
        L["mixer"].pop("_rel_rows", None)
    return c


def write_folder(path: Path, cfg: dict, weights: Dict[str, torch.Tensor]) -> Path:
    from safetensors.torch import save_file

    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(clean_config(cfg)))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(path / "model.safetensors"))
    return path
