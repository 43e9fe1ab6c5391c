"""Host-side parts of the Taruvik design: configuration, layer runs of a looped span, rotation frequencies, checkpoint packing."""
import json
import math

import pytest
import torch

from tests import taruvik_oracle as O
from tests.taruvik_util import make_config, make_weights, mixer_cfg, moe_cfg, write_folder


def test_config_and_layer_runs():
    from mistral_inference_b200.args import LayeredArgs, LatentAttentionArgs, MoeFfArgs

    cfg = make_config(layers=[(mixer_cfg(), moe_cfg()), (mixer_cfg(), None), (mixer_cfg(), moe_cfg(count=0)), (mixer_cfg(), None)], loop=(1, 3, 3))
    a = LayeredArgs.from_dict(json.loads(json.dumps(cfg)))
    assert a.norm == "layer" and a.post_norm and a.embedding_scale == 1.0
    assert a.layer_runs() == [0, 1, 2, 1, 2, 1, 2, 3] == O.layer_schedule(cfg)
    assert isinstance(a.layers[0].mixer, LatentAttentionArgs) and isinstance(a.layers[0].mlp, MoeFfArgs) and a.layers[1].mlp is None
    assert (a.layers[0].mlp.routed, a.layers[0].mlp.groups, a.layers[0].mlp.keep) == (8, 4, 2)
    assert (a.layers[2].mlp.groups, a.layers[2].mlp.keep) == (1, 1)
    cfg.pop("loop")
    assert LayeredArgs.from_dict(cfg).layer_runs() == [0, 1, 2, 3]
    with pytest.raises(ValueError):
        LayeredArgs.from_dict({**cfg, "architecture": "Nothing"})
    bad = make_config(layers=[(mixer_cfg(), moe_cfg(experts=6, identity=1, count=2))])
    with pytest.raises(AssertionError):
        LayeredArgs.from_dict(bad)    # 7 routed outputs do not form 2 equal groups


@pytest.mark.parametrize("rot", [{"base": 1000.0, "dims": 8}, {"base": 5e5, "dims": 32, "scaling": {"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0}},
                                 {"base": 10000.0, "dims": 4, "scaling": {"factor": 8.0, "original": 8, "fast": 2.0, "slow": 0.5}}])
def test_rotation_frequencies(rot):
    from mistral_inference_b200.args import LatentAttentionArgs
    from mistral_inference_b200.rope import scaled_frequencies

    a = LatentAttentionArgs.from_dict(mixer_cfg(rot=rot, rot_dim=rot["dims"]))
    f, mag = scaled_frequencies(a.rot_dims, a.rot_base, a.rot_scaling)
    fo, mo = O.yarn_frequencies(rot)
    torch.testing.assert_close(f, fo, rtol=1e-12, atol=0)
    assert mag == pytest.approx(mo)
    if "scaling" not in rot:
        assert mag == 1.0 and f[1].item() == pytest.approx(rot["base"] ** (-2.0 / rot["dims"]))
    else:  # the slowest pair is divided by the factor, the fastest is not (for these tables)
        assert f[0].item() == pytest.approx(1.0) and f[-1].item() == pytest.approx(fo[-1].item())
        assert mag == pytest.approx(0.1 * math.log(rot["scaling"]["factor"]) + 1)


def test_checkpoint_packing(tmp_path):
    from mistral_inference_b200.registry import architecture_of, load_model

    cfg = make_config(layers=[(mixer_cfg(), moe_cfg()), (mixer_cfg(heads=2), None)], loop=(0, 1, 2))
    w = make_weights(cfg, 3)
    folder = write_folder(tmp_path / "m", cfg, w)
    assert architecture_of(folder) == "Taruvik"
    m = load_model(folder, device="cpu", dtype=torch.float32)
    assert set(m.checkpoint_keys()) == set(w)
    ff, mx = m.layers[0].mlp, m.layers[0].mix
    a = ff.a
    assert torch.equal(ff.w13.view(a.experts, a.ff, 2, 40)[4, :, 0], w["l0.mlp.e4.gate"]) and torch.equal(ff.w13[2 * a.ff * 2 + 1], w["l0.mlp.e2.up"][0])
    assert torch.equal(ff.w2[:, 3 * a.ff: 4 * a.ff], w["l0.mlp.e3.down"])
    assert torch.equal(mx.w_in[: mx.a.q_rank], w["l0.mix.dq"]) and torch.equal(mx.w_in[-mx.a.heads:], w["l0.mix.g"])
    assert torch.equal(m.layers[1].norm1b.bias, w["l1.norm1b.b"]) and m.layers[1].norm2 is None
    cache = m.make_cache(2, 16)   # one ring per layer run, latent rows, no value ring
    assert len(cache.cache_k) == 3 and cache.cache_k[0].shape == (2, 16, 1, mx.a.kv_rank + mx.a.rot_dim) and cache.cache_v[0].shape[-1] == 0
    w.pop("l0.mlp.e1.up")
    write_folder(tmp_path / "n", cfg, w)
    with pytest.raises(AssertionError):
        load_model(tmp_path / "n", device="cpu", dtype=torch.float32)


def test_oracle_router_is_what_it_says():
    """The oracle's router on a hand-made case: the best group is chosen by score + correction, the weights are the plain scores."""
    W = {"router": torch.eye(4) * 2.0, "correction": torch.tensor([0.0, 0.0, 0.0, 0.6])}
    r = {"experts": 3, "identity": 1, "top": 1, "groups": {"count": 2, "keep": 1}}
    h = torch.tensor([[3.0, 0.0, 0.0, 0.0]])   # output 0 has by far the largest score, but output 3's correction wins the choice
    s = torch.softmax(h @ W["router"].T, -1)
    out = O.route(h, {"p.router": W["router"], "p.correction": W["correction"]}, "p.", r)
    if s[0, 3] + 0.6 > s[0, 0]:
        assert out[0, 3] == s[0, 3] and out[0, :3].eq(0).all()
    else:
        assert out[0, 0] == s[0, 0]
