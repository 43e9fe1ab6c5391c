"""Host-side parts of the layered decoder: config parsing, distance buckets, cache specs / slots / retire, registry."""
import json

import pytest
import torch

from mistral_inference_b200.args import LayeredArgs
from mistral_inference_b200.cache import BufferCache, LayerCacheSpec
from mistral_inference_b200.transformer_layers import distance_buckets
from tests import fesenex_oracle as O
from tests.fesenex_util import make_config


@pytest.mark.parametrize("rows,far", [(30, 200.0), (8, 64.0), (16, 1000.0), (4, 3.0), (64, 33.0)])
def test_distance_buckets_match_the_oracle(rows, far):
    tab = distance_buckets(rows, far)
    assert tab[-1] == rows - 1 and all(b < rows - 1 for b in tab[:-1])
    for n in range(len(tab) + 50):
        assert (tab[n] if n < len(tab) else rows - 1) == O.rel_bucket(n, rows, far), n
    assert tab[: rows // 2] == list(range(rows // 2))


def test_config_parsing_reads_every_constant():
    cfg = make_config(width=48, vocab=50, layers=[("attention", dict(heads=4, kv_heads=2, dim=16, vdim=8, v_mix=True)),
                                                 ("lightning", dict(heads=2, dim=16, vdim=8), None),
                                                 ("attention", dict(heads=4, kv_heads=2, dim=16, vdim=8, v_mix=True, q_temp=None))])
    a = LayeredArgs.from_dict(json.loads(json.dumps(cfg)))
    assert a.width == 48 and a.vocab == 50 and len(a.layers) == 3
    assert a.layers[0].mixer.temp_every == cfg["layers"][0]["mixer"]["q_temp"]["every"]
    assert a.layers[1].mlp is None and a.layers[1].mixer.decay == cfg["layers"][1]["mixer"]["decay"]
    assert a.layers[2].mixer.temp_every == 0
    with pytest.raises(ValueError):
        LayeredArgs.from_dict({**cfg, "layers": [{"type": "conv", "mixer": {}, "mlp": None}]})


def test_cache_specs_slots_and_retire():
    specs = [LayerCacheSpec(kind="ring", n_kv_heads=2, k_dim=8, v_dim=4), LayerCacheSpec(kind="state", state_shape=(3, 8, 4))]
    c = BufferCache(2, 3, 10, 0, 0, None, layer_specs=specs)
    assert c.cache_k[0].shape == (3, 10, 2, 8) and c.cache_v[0].shape == (3, 10, 2, 4)
    assert c.cache_state[1].shape == (3, 3, 8, 4) and c.cache_state[1].dtype == torch.float32 and 1 not in c.cache_k
    md = c.get_input_metadata([2, 4, 1])
    assert md[0].slots.tolist() == [0, 1, 2]
    assert md[0].cache_rows.tolist() == [0, 1, 10, 11, 12, 13, 20]
    c.update_seqlens([2, 4, 1])
    c.retire([1])                       # the middle one ends: the others keep rows 0 and 2
    md = c.get_input_metadata([1, 1])
    assert md[1].slots.tolist() == [0, 2] and md[0].positions.tolist() == [2, 1] and md[0].cache_rows.tolist() == [2, 21]
    c.update_seqlens([1, 1])
    c.retire([0, 1])
    c.reset()
    md = c.get_input_metadata([3])      # a new batch gets row 0 again, from position 0
    assert md[0].slots.tolist() == [0] and md[0].seqpos.tolist() == [0]
    assert c.get_view(1, md[1]).state is c.cache_state[1]


def test_registry_picks_the_class_by_the_folder(tmp_path):
    from mistral_inference_b200 import registry

    (tmp_path / "a").mkdir()
    (tmp_path / "a" / "config.json").write_text(json.dumps({"architecture": "Fesenex"}))
    (tmp_path / "b").mkdir()
    (tmp_path / "b" / "params.json").write_text("{}")
    (tmp_path / "c").mkdir()
    (tmp_path / "c" / "config.json").write_text(json.dumps({"architecture": "nope"}))
    assert registry.architecture_of(tmp_path / "a") == "Fesenex"
    assert registry.architecture_of(tmp_path / "b") == "transformer"
    with pytest.raises(ValueError):
        registry.architecture_of(tmp_path / "c")


def test_hybrid_binding_matches_the_header():
    """Every function the header declares is bound with as many arguments, and nothing else is bound."""
    import re
    from pathlib import Path

    from mistral_inference_b200 import _abi_hybrid

    text = (Path(__file__).resolve().parent.parent / "include" / "mistral_b200_hybrid.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    decl = {m.group(1): m.group(2) for m in re.finditer(r"\b(mbh_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S)}
    assert set(decl) == set(_abi_hybrid._SIGNATURES)
    for name, params in decl.items():
        n = 0 if params.strip() == "void" else params.count(",") + 1
        assert n == len(_abi_hybrid._SIGNATURES[name][1]), name
