"""The layered decoder on the GPU against the plain fp32 statement in tests/fesenex_oracle.py: every mechanism alone, then
whole models of several shapes through the cache (prompt against token-by-token decoding, portions, ragged batches, rows
that are reused) and greedy generation through `generate()`.  fp32 runs are compared tightly, bf16 runs by an error norm."""
import math

import pytest
import torch

from tests import fesenex_oracle as O
from tests.fesenex_util import clean_config, make_config, make_weights, write_folder

pytestmark = pytest.mark.gpu
DEV = "cuda"

MIXED = [("attention", dict(v_mix=True)), ("lightning", {}, None), ("attention", dict(v_mix=True)), ("attention", dict(v_mix=False, q_temp=None))]
SHAPES = {
    "mixed": dict(width=48, vocab=64, layers=MIXED),
    # heads == kv_heads, one kv head, value size above key size, sizes that are no multiple of 8, lightning first, no feed-forward last
    "odd": dict(width=44, vocab=37, layers=[("lightning", dict(heads=3, dim=20, vdim=36)), ("attention", dict(heads=3, kv_heads=3, dim=12, vdim=20, _rel_rows=6, bias_max=9)),
                                            ("attention", dict(heads=4, kv_heads=1, dim=24, vdim=40, v_mix=True, _rel_rows=12, bias_max=100), None)]),
    "wide": dict(width=96, vocab=80, layers=[("attention", dict(heads=6, kv_heads=2, dim=64, vdim=32, v_mix=True, _rel_rows=24, bias_max=200, q_temp={"coef": 0.7, "every": 16})),
                                             ("lightning", dict(heads=2, dim=64, vdim=64)), ("lightning", dict(heads=1, dim=96, vdim=16), None),
                                             ("attention", dict(heads=6, kv_heads=2, dim=64, vdim=32, v_mix=True, _rel_rows=24, bias_max=200))]),
}


def _model(tmp_path, name, dtype, seed=0):
    from mistral_inference_b200.registry import load_model

    cfg = make_config(**SHAPES[name])
    w = make_weights(cfg, seed)
    m = load_model(write_folder(tmp_path / name, cfg, w), device=DEV, dtype=dtype)
    return m, clean_config(cfg), w


def _tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def _close(got, ref, dtype, what=""):
    got, ref = got.float().cpu(), ref.float()
    if dtype == torch.float32:
        torch.testing.assert_close(got, ref, rtol=2e-4, atol=2e-4, msg=lambda m: f"{what}: {m}")
    else:
        err = (got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt().clamp_min(1e-6)
        assert err < 0.04, f"{what}: relative rms error {err:.4f}"


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 10, 7), (3, 33, 40), (8, 64, 64), (5, 50, 296), (4, 37, 23), (9, 50, 24), (70, 130, 100), (200, 96, 328), (256, 256, 128), (130, 384, 64)])
def test_linear_epilogues(dtype, M, N, K):
    from mistral_inference_b200 import _abi_hybrid as h

    g = torch.Generator().manual_seed(M * N + K)
    x = torch.randn(M, K, generator=g).to(dtype).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(dtype).to(DEV)
    b = torch.randn(N, generator=g).to(dtype).to(DEV)
    y = x.float().cpu() @ w.float().cpu().T + b.float().cpu()
    n_act = N // 2
    ref = y.clone()
    ref[:, :n_act] = torch.nn.functional.silu(y[:, :n_act])
    _close(h.linear(x, w, b, n_act=n_act), ref, dtype, "store")
    _close(h.linear(x, w, b, epi=h.EPI_F32), y, dtype, "fp32 out")
    res = torch.randn(M, N, generator=g).to(DEV)
    want = res.cpu() + y
    h.linear(x, w, b, epi=h.EPI_RESIDUAL, residual=res)
    _close(res, want, dtype, "residual")
    if N % 2 == 0:
        yy = x.float().cpu() @ w.float().cpu().T
        gate, up = yy[:, 0::2].clamp(max=0.7), yy[:, 1::2].clamp(-0.7, 0.7)
        _close(h.linear(x, w, epi=h.EPI_GLU, limit=0.7, alpha=1.702), gate * torch.sigmoid(1.702 * gate) * (up + 1), dtype, "glu")


def test_rmsnorm_and_embedding():
    from mistral_inference_b200 import _abi_hybrid as h

    x = torch.randn(5, 44, device=DEV) * 3
    w = torch.randn(44, device=DEV)
    _close(h.rmsnorm(x, w, 1e-2), O.norm(x.cpu(), w.cpu(), 1e-2), torch.float32)
    tab = torch.randn(9, 44, device=DEV)
    tok = torch.tensor([3, 8, 0], device=DEV)
    _close(h.embed_scale(tok, tab, 2.5), tab.cpu()[tok.cpu()] * 2.5, torch.float32)


def _one_layer(kind, mix, n, seed=1, mlp=None):
    cfg = make_config(width=32, vocab=16, layers=[(kind, mix, mlp)])
    return clean_config(cfg), make_weights(cfg, seed, dtype=torch.float32)


def _run_layers(tmp_path, cfg, w, toks, dtype=torch.float32, portions=None):
    """Residual stream after the last layer, through the product path, the prompt cut into `portions`."""
    from mistral_inference_b200.registry import load_model

    m = load_model(write_folder(tmp_path / "m", cfg, w), device=DEV, dtype=dtype)
    cache = m.make_cache(1, len(toks))
    outs, o = [], 0
    for p in portions or [len(toks)]:
        outs.append(m.hidden(torch.tensor(toks[o:o + p], device=DEV), [p], cache).clone())
        o += p
    return torch.cat(outs)


@pytest.mark.parametrize("mix", [dict(heads=4, kv_heads=2, dim=16, vdim=8), dict(heads=2, kv_heads=2, dim=8, vdim=24, q_temp=None),
                                 dict(heads=6, kv_heads=1, dim=20, vdim=4, _rel_rows=4, bias_max=5, q_temp={"coef": 1.0, "every": 1})])
def test_attention_mixer_alone(tmp_path, mix):
    cfg, w = _one_layer("attention", mix, 40, mlp=None)
    toks = _tokens(cfg, 40, 3)
    lay = []
    O.forward(cfg, w, toks, lay)
    _close(_run_layers(tmp_path, cfg, w, toks), lay[0], torch.float32)


@pytest.mark.parametrize("mix", [dict(heads=2, dim=16, vdim=8), dict(heads=1, dim=40, vdim=40, decay=[0.999]), dict(heads=3, dim=8, vdim=70, decay=[0.2, 1.0, 0.9])])
def test_lightning_mixer_alone_and_its_state(tmp_path, mix):
    cfg, w = _one_layer("lightning", mix, 50, mlp=None)
    toks = _tokens(cfg, 50, 4)
    lay = []
    O.forward(cfg, w, toks, lay)
    _close(_run_layers(tmp_path, cfg, w, toks), lay[0], torch.float32, "whole")
    _close(_run_layers(tmp_path, cfg, w, toks, portions=[17, 2, 16, 1, 14]), lay[0], torch.float32, "portions carry the state")


def test_feed_forward_alone(tmp_path):
    cfg, w = _one_layer("lightning", dict(heads=1, dim=8, vdim=8), 12, mlp={"ff": 24, "limit": 0.3})
    toks = _tokens(cfg, 12, 5)
    lay = []
    O.forward(cfg, w, toks, lay)
    _close(_run_layers(tmp_path, cfg, w, toks), lay[0], torch.float32)


def test_far_key_and_bucket_edges_stand_out(tmp_path):
    """One query/key pair far back is scaled so that its score dominates: the output must be that key's value, at distances
    on both sides of every bucket edge and far beyond the last one, for a prompt and for decoded tokens."""
    mix = dict(heads=2, kv_heads=1, dim=8, vdim=8, _rel_rows=8, bias_max=24, q_temp=None, scale=1.0)
    cfg, w = _one_layer("attention", mix, 0, mlp=None)
    # a bias table that alone decides the winner: bucket b of head 0 gets 30 * [b == target]
    from mistral_inference_b200.transformer_layers import distance_buckets
    tab = distance_buckets(8, 24)
    edges = sorted({n for n in range(1, len(tab)) if tab[n] != tab[n - 1]} | {len(tab) - 1, len(tab) + 40})
    n = len(tab) + 60
    toks = _tokens(cfg, n, 6)
    for target in range(8):
        w["l0.mix.rel"] = torch.zeros(8, 2)
        w["l0.mix.rel"][target, 0] = 30.0
        w["l0.mix.rel"][7 - target, 1] = 30.0
        lay = []
        O.forward(cfg, w, toks, lay)
        _close(_run_layers(tmp_path, cfg, w, toks), lay[0], torch.float32, f"prompt, bucket {target}")
        _close(_run_layers(tmp_path, cfg, w, toks, portions=[n - 40] + [1] * 40), lay[0], torch.float32, f"decoded, bucket {target}")
    assert edges  # the distances above are all inside the sequence: n > last edge + 40


# ----------------------------------------------------------------------------- whole models through the cache
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(SHAPES))
def test_whole_prompt_matches_the_oracle(tmp_path, name, dtype):
    m, cfg, w = _model(tmp_path, name, dtype)
    toks = _tokens(cfg, 70, 1)
    ref = O.forward(cfg, w, toks)
    _close(m.forward(torch.tensor(toks, device=DEV), [len(toks)], None), ref, dtype)


@pytest.mark.parametrize("name", list(SHAPES))
def test_prefill_decode_and_portions_agree(tmp_path, name):
    m, cfg, w = _model(tmp_path, name, torch.float32)
    toks = _tokens(cfg, 61, 2)
    ref = O.forward(cfg, w, toks)
    for portions in ([61], [1] * 61, [2] * 30 + [1], [33, 2, 7, 19], [60, 1], [1, 60]):
        cache = m.make_cache(1, 61)
        outs, o = [], 0
        for p in portions:
            outs.append(m.forward(torch.tensor(toks[o:o + p], device=DEV), [p], cache))
            o += p
        _close(torch.cat(outs), ref, torch.float32, f"{name} {portions[:4]}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_batch_retire_and_row_reuse(tmp_path, dtype):
    """Three unequal requests start together and decode together, the shorter ones end earlier; then a new batch takes the same
    rows (with the earlier state and keys still in memory) and must not see them."""
    m, cfg, w = _model(tmp_path, "mixed", dtype)
    lens, starts = [9, 30, 17], [5, 22, 1]         # total length, tokens given in the first step
    reqs = [_tokens(cfg, n, 10 + i) for i, n in enumerate(lens)]
    refs = [O.forward(cfg, w, r) for r in reqs]
    cache = m.make_cache(3, 32)
    for round_ in range(2):
        cache.reset()
        cache.init_kvseqlens(3)
        live = [0, 1, 2]
        at = list(starts)
        flat = [t for i in live for t in reqs[i][: at[i]]]
        out = m.forward(torch.tensor(flat, device=DEV), [at[i] for i in live], cache)
        o = 0
        for i in live:
            _close(out[o:o + at[i]], refs[i][: at[i]], dtype, f"round {round_} prompt {i}")
            o += at[i]
        while live:
            gone = [k for k, i in enumerate(live) if at[i] == lens[i]]
            if gone:
                cache.retire(gone)
                live = [i for k, i in enumerate(live) if k not in gone]
                continue
            out = m.forward(torch.tensor([reqs[i][at[i]] for i in live], device=DEV), [1] * len(live), cache)
            for k, i in enumerate(live):
                _close(out[k], refs[i][at[i]], dtype, f"round {round_} request {i} token {at[i]}")
                at[i] += 1
        reqs = reqs[::-1]; refs = refs[::-1]; lens = lens[::-1]; starts = [3, 8, 2]  # other requests in the same rows


def test_long_decoding_keeps_the_state(tmp_path):
    m, cfg, w = _model(tmp_path, "odd", torch.float32)
    toks = _tokens(cfg, 330, 7)
    ref = O.forward(cfg, w, toks)
    cache = m.make_cache(1, 330)
    out = [m.forward(torch.tensor(toks[:10], device=DEV), [10], cache)]
    for t in toks[10:]:
        out.append(m.forward(torch.tensor([t], device=DEV), [1], cache))
    _close(torch.cat(out), ref, torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_generate(tmp_path, dtype):
    from mistral_inference_b200.generate import generate

    m, cfg, w = _model(tmp_path, "mixed", dtype)
    m.args.max_batch_size = 2
    prompts = [_tokens(cfg, 12, 20), _tokens(cfg, 7, 21)]
    got, lps = generate(prompts, m, max_tokens=6, temperature=0.0, chunk_size=6)
    for p, g, lp in zip(prompts, got, lps):
        seq = list(p)
        for k, tok in enumerate(g):
            logits = O.forward(cfg, w, seq)[-1]
            top = torch.topk(logits, 2).values
            if dtype == torch.float32 or top[0] - top[1] > 0.05:   # a near tie may fall either way in bf16
                assert tok == int(logits.argmax()), (k, tok)
            seq.append(tok)
        assert len(lp) == len(p) - 1 + len(g)
        ref_lp = torch.log_softmax(O.forward(cfg, w, seq[:-1]), -1)
        want = torch.tensor([ref_lp[i, seq[i + 1]] for i in range(len(seq) - 1)])
        assert (torch.tensor(lp) - want).abs().max() < (1e-3 if dtype == torch.float32 else 0.15)


# ----------------------------------------------------------------------------- attention kernels against each other and the oracle
def _attn_case(dtype, lens, past, H, G, d, e, W, seed=0):
    """A ragged batch with `past[b]` cached tokens and `lens[b]` new ones; returns the kernel inputs and a dense reference."""
    from mistral_inference_b200.cache import BufferCache, LayerCacheSpec

    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    cache = BufferCache(1, B + 1, W, 0, 0, None, layer_specs=[LayerCacheSpec(kind="ring", n_kv_heads=G, k_dim=d, v_dim=e)]).to(DEV, dtype)
    cache.cache_k[0].copy_(torch.randn(cache.cache_k[0].shape, generator=g))
    cache.cache_v[0].copy_(torch.randn(cache.cache_v[0].shape, generator=g))
    cache.init_kvseqlens(B)
    cache._rows = list(range(1, B + 1))   # not the identity: slot b + 1
    cache.update_seqlens(past)
    md = cache.get_input_metadata(lens)[0]
    T = sum(lens)
    q = torch.randn(T, H * d, generator=g).to(dtype).to(DEV)
    tab = (torch.randn(11, H, generator=g) * 2).to(DEV)
    scale = 0.3
    ref = torch.zeros(T, H, e)
    Kc, Vc, qq = cache.cache_k[0].float().cpu(), cache.cache_v[0].float().cpu(), q.float().cpu().view(T, H, d)
    t = 0
    for b in range(B):
        for i in range(lens[b]):
            pos = past[b] + i
            for hh in range(H):
                kv = hh // (H // G)
                s = (Kc[b + 1, : pos + 1, kv] @ qq[t, hh]) * scale + tab.cpu()[torch.clamp(pos - torch.arange(pos + 1), max=10), hh]
                ref[t, hh] = torch.softmax(s, 0) @ Vc[b + 1, : pos + 1, kv]
            t += 1
    return cache, md, q, tab, scale, ref.view(T, H * e)


@pytest.mark.parametrize("d,e", [(64, 32), (32, 32), (128, 128), (64, 128)])
def test_tensor_core_prompt_attention(d, e):
    from mistral_inference_b200 import _abi_hybrid as h

    H, G, W = 4, 2, 400
    lens, past = [64, 130, 17, 1, 65], [70, 0, 200, 5, 63]    # whole tiles, partial tiles, portions that start inside a tile of keys
    cache, md, q, tab, scale, ref = _attn_case(torch.bfloat16, lens, past, H, G, d, e, W)
    out = torch.empty(q.shape[0], H * e, dtype=torch.bfloat16, device=DEV)
    h.attn_bias(q, cache.cache_k[0], cache.cache_v[0], tab, md.positions, md.q_start, md.slots, out, len(lens), W, H, G, d, e, scale,
                n_tiles=sum((n + 63) // 64 for n in lens))
    err = (out.float().cpu() - ref).abs().max() / ref.abs().max()
    assert err < 0.02, err


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_exact_attention_with_split_keys(dtype, splits):
    from mistral_inference_b200 import _abi_hybrid as h

    H, G, d, e, W = 6, 3, 24, 40, 1500
    lens, past = [1, 1, 1, 2], [513, 0, 1499, 127]            # first token, the last ring row, chunk edges of the kernel
    cache, md, q, tab, scale, ref = _attn_case(dtype, lens, past, H, G, d, e, W, seed=3)
    out = torch.empty(q.shape[0], H * e, dtype=dtype, device=DEV)
    h.attn_bias(q, cache.cache_k[0], cache.cache_v[0], tab, md.positions, md.q_start, md.slots, out, len(lens), W, H, G, d, e, scale, splits=splits)
    err = (out.float().cpu() - ref).abs().max() / ref.abs().max()
    assert err < (1e-4 if dtype == torch.float32 else 0.02), err


def test_trace_runner_replays_a_schedule(tmp_path):
    """bin/trace_run on a small folder: a ragged batch that starts together, decodes, loses its shorter request, then a second
    batch in the same rows; the files it writes hold the oracle's logits at the places asked for."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    cfg = make_config(**SHAPES["mixed"])
    w = make_weights(cfg, 5)
    folder = write_folder(tmp_path / "model", cfg, w)
    cfg = clean_config(cfg)
    a, b, c = _tokens(cfg, 20, 31), _tokens(cfg, 9, 32), _tokens(cfg, 26, 33)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:18], "want": [0, 17]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[18:19], "want": []}, {"id": "b", "tokens": b[8:9], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[19:20], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "c", "tokens": c[:24], "want": [23]}], "end": []},
             {"step": 4, "entries": [{"id": "c", "tokens": c[24:25], "want": [0]}], "end": []},
             {"step": 5, "entries": [{"id": "c", "tokens": c[25:26], "want": [0]}], "end": ["c"]}]
    out = tmp_path / "out"
    exe = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    r = subprocess.run([sys.executable, str(exe), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.split("\n") if ln.startswith("done")] == [f"done {i}" for i in range(6)]
    ra, rb, rc = (O.forward(cfg, w, t) for t in (a, b, c))
    want = {0: torch.stack([ra[0], ra[17], rb[7]]), 1: rb[8:9], 2: ra[19:20], 3: rc[23:24], 4: rc[24:25], 5: rc[25:26]}
    for n, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        _close(got, ref, torch.float32, f"step {n}")
