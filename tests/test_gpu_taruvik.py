"""The Taruvik design on the GPU against the plain fp32 statement in tests/taruvik_oracle.py: every mechanism alone (layer norm,
gated Linear with routing weights, router, experts dense and sparse, latent attention), then whole models of several shapes
through the cache: prompts against token-by-token decoding, portions, ragged batches, reused rows, far keys, long decoding,
looped layers, and greedy generation through `generate()`.  fp32 runs are compared tightly, bf16 runs by an error norm."""
import math

import pytest
import torch

from tests import taruvik_oracle as O
from tests.taruvik_util import f32, make_config, make_weights, mixer_cfg, moe_cfg, write_folder

pytestmark = pytest.mark.gpu
DEV = "cuda"

SHAPES = {
    # three heads, sizes that are no multiple of 8, rotation over part of the rotated entries, a loop over the middle layers
    "odd": dict(width=40, vocab=50, loop=(1, 3, 3),
                layers=[(mixer_cfg(), moe_cfg()),
                        (mixer_cfg(heads=2, dim=10, rot_dim=12, vdim=6, q_rank=14, kv_rank=22, rot={"base": 50.0, "dims": 8}), None),
                        (mixer_cfg(heads=5, dim=4, rot_dim=4, vdim=9, rot={"base": 10000.0, "dims": 4, "scaling": {"factor": 8.0, "original": 8, "fast": 2.0, "slow": 0.5}}),
                         moe_cfg(ff=10, experts=5, top=2, identity=0, count=0)),
                        (mixer_cfg(heads=1, kv_rank=64), moe_cfg(ff=16, experts=3, top=4, identity=5, count=2, keep=2))]),
    # one expert per token, one group kept of many, the loop is the whole model and runs once, no feed-forward in the first layer
    "single": dict(width=64, vocab=33, loop=(0, 2, 1),
                   layers=[(mixer_cfg(heads=4, dim=16, rot_dim=16, vdim=16, q_rank=32, kv_rank=32, rot={"base": 100.0, "dims": 16}), None),
                           (mixer_cfg(heads=4, dim=16, rot_dim=16, vdim=16, q_rank=32, kv_rank=32), moe_cfg(ff=32, experts=9, top=1, identity=3, count=6, keep=1))]),
    # a latent wider than 256 (the wide attention kernel), no loop; both router groups stay (in bf16 a near tie between two GROUPS
    # would exchange a token's whole set of experts; the choice among groups is covered in fp32 and by test_router)
    "wide": dict(width=96, vocab=70, layers=[(mixer_cfg(heads=2, dim=24, rot_dim=32, vdim=40, q_rank=48, kv_rank=288, rot={"base": 500.0, "dims": 32}),
                                              moe_cfg(ff=40, experts=8, top=3, identity=0, count=2, keep=2))] * 2),
}


def _model(tmp_path, name, dtype, seed=0, **over):
    from mistral_inference_b200.registry import load_model

    cfg = make_config(**{**SHAPES[name], **over})
    w = make_weights(cfg, seed)
    m = load_model(write_folder(tmp_path / name, cfg, w), device=DEV, dtype=dtype)
    if dtype == torch.bfloat16:  # the oracle sees the rounded weights
        w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    return m, cfg, f32(w)


def _tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def _close(got, ref, dtype, what=""):
    got, ref = got.float().cpu(), ref.float().cpu()
    if dtype == torch.float32:
        torch.testing.assert_close(got, ref, rtol=3e-4, atol=3e-4, msg=lambda m: f"{what}: {m}")
    else:
        # per token: most are within bf16 rounding.  The activations that reach a router differ from the fp32 oracle's by a percent
        # or so, which turns a near tie between two experts the other way for a few tokens in a hundred, whatever the router's
        # gain; such a token is off by 0.1 to 0.2 with these weights.  A fault of a kernel or the cache moves most tokens.
        got, ref = got.reshape(-1, got.shape[-1]), ref.reshape(-1, ref.shape[-1])
        err = (got - ref).pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt().clamp_min(1e-6)
        assert err.median() < 0.04, f"{what}: median relative rms error {err.median():.4f}"
        assert int((err > 0.2).sum()) <= max(1, len(err) // 10), f"{what}: {int((err > 0.2).sum())} of {len(err)} tokens are far off ({err.max():.3f})"


# ----------------------------------------------------------------------------- mechanisms alone
def test_layer_norm_and_added_embedding():
    from mistral_inference_b200 import _abi_hybrid as h

    x = torch.randn(7, 44, device=DEV) * 3 + 5   # a mean well away from 0: mean of squares minus square of mean would lose digits
    w, b = torch.randn(44, device=DEV), torch.randn(44, device=DEV)
    ref = O.layer_norm(x.cpu(), w.cpu(), b.cpu(), 1e-3)
    _close(h.layernorm(x, w, b, 1e-3), ref, torch.float32)
    acc = torch.randn(7, 44, device=DEV)
    want = acc.cpu() + ref
    h.layernorm(x, w, b, 1e-3, add_to=acc)
    _close(acc, want, torch.float32)
    _close(h.layernorm(x, w.bfloat16(), b.bfloat16(), 1e-3), O.layer_norm(x.cpu(), w.bfloat16().float().cpu(), b.bfloat16().float().cpu(), 1e-3), torch.bfloat16)
    tab = torch.randn(9, 44, device=DEV)
    tok = torch.tensor([3, 8, 0, 3, 1, 1, 7], device=DEV)
    want = acc.cpu() + tab.cpu()[tok.cpu()]
    h.embed_add(tok, tab, 1.0, acc)
    _close(acc, want, torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,F,K,group", [(1, 12, 20, 4), (5, 30, 44, 10), (8, 32, 64, 8), (70, 66, 100, 22), (200, 128, 64, 32)])
def test_gated_linear_with_routing_weights(dtype, M, F, K, group):
    from mistral_inference_b200 import _abi_hybrid as h

    g = torch.Generator().manual_seed(M + F)
    x = torch.randn(M, K, generator=g).to(dtype).to(DEV)
    w = (torch.randn(2 * F, K, generator=g) / math.sqrt(K)).to(dtype).to(DEV)
    rs = torch.rand(M, F // group, generator=g)
    rs[rs < 0.4] = 0.0
    y = x.float().cpu() @ w.float().cpu().T
    ref = torch.nn.functional.silu(y[:, 0::2]) * y[:, 1::2]
    _close(h.linear_swiglu(x, w), ref, dtype, "plain")
    _close(h.linear_swiglu(x, w, rowscale=rs.to(DEV), group=group), ref * rs.repeat_interleave(group, 1), dtype, "scaled")


ROUTERS = [dict(experts=6, top=3, identity=2, count=4, keep=2), dict(experts=5, top=2, identity=0, count=0), dict(experts=3, top=4, identity=5, count=2, keep=2),
           dict(experts=9, top=1, identity=3, count=6, keep=1), dict(experts=40, top=6, identity=8, count=8, keep=3), dict(experts=7, top=7, identity=0, count=1, keep=1)]


@pytest.mark.parametrize("r", ROUTERS)
@pytest.mark.parametrize("neg", [False, True])
def test_router(r, neg):
    """Dense weights and chosen pairs against the oracle; `neg` makes every choice score negative (a dropped group must count
    as minus infinity, not 0)."""
    from mistral_inference_b200 import _abi_hybrid as h

    cfg = make_config(width=32, layers=[(mixer_cfg(), moe_cfg(ff=8, **r))])
    w = make_weights(cfg, 5)
    if neg:
        w["l0.mlp.correction"] = w["l0.mlp.correction"] - 2.0
    x = torch.randn(50, 32, generator=torch.Generator().manual_seed(1))
    ref = O.route(x, w, "l0.mlp.", cfg["layers"][0]["mlp"]["router"])
    a = cfg["layers"][0]["mlp"]["router"]
    gr = a.get("groups") or {"count": 1, "keep": 1}
    dense, idx, wsel = h.moe_route(x.to(DEV), w["l0.mlp.router"].to(DEV), w["l0.mlp.correction"].to(DEV), gr["count"], gr["keep"], a["top"])
    assert ((dense.cpu() > 0) == (ref > 0)).all(), "another set of experts"
    _close(dense, ref, torch.float32)
    assert (dense.cpu() > 0).sum(1).eq(a["top"]).all()
    _close(torch.gather(dense, 1, idx.long()), wsel, torch.float32, "pairs agree with the dense form")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("r", ROUTERS[:5])
def test_experts_dense_and_sparse(dtype, r):
    from mistral_inference_b200.args import MoeFfArgs
    from mistral_inference_b200.transformer_layers import MoeFeedForward

    width = 40
    cfg = make_config(width=width, layers=[(mixer_cfg(), moe_cfg(ff=12, **r))])
    w = {k: v.to(dtype) for k, v in make_weights(cfg, 3).items()}
    ff = MoeFeedForward(width, MoeFfArgs.from_dict(cfg["layers"][0]["mlp"])).to(dtype).to(DEV)
    for k, v in w.items():
        if k.startswith("l0.mlp."):
            assert ff.assign(k[len("l0.mlp."):], lambda dst: dst.copy_(v)), k
    x = torch.randn(30, width, generator=torch.Generator().manual_seed(2)).to(dtype)
    ref = O.moe(x.float(), f32(w), "l0.mlp.", cfg["layers"][0]["mlp"])
    for sparse in (0, 1000):
        ff.sparse_max_tokens = sparse
        acc = torch.zeros(30, width, device=DEV)
        ff.run(x.to(DEV), acc)
        _close(acc, ref, dtype, "sparse" if sparse else "dense")


def _hidden(m, toks, portions=None, taps=None):
    cache = m.make_cache(1, len(toks))
    outs, o = [], 0
    for p in portions or [len(toks)]:
        outs.append(m.hidden(torch.tensor(toks[o:o + p], device=DEV), [p], cache).clone())
        o += p
    return torch.cat(outs)


@pytest.mark.parametrize("mix", [mixer_cfg(), mixer_cfg(heads=1, dim=7, rot_dim=6, vdim=5, q_rank=9, kv_rank=11, rot={"base": 20.0, "dims": 4}),
                                 mixer_cfg(heads=6, dim=32, rot_dim=16, vdim=32, q_rank=16, kv_rank=300, scale=1.5, rot={"base": 1e4, "dims": 16}),
                                 # 12 and 20 heads: the decode kernel gives a warp two and four heads
                                 mixer_cfg(heads=12, dim=8, rot_dim=8, vdim=8, q_rank=16, kv_rank=24, rot={"base": 100.0, "dims": 8}),
                                 mixer_cfg(heads=20, dim=6, rot_dim=4, vdim=10, q_rank=12, kv_rank=18, scale=0.8, rot={"base": 100.0, "dims": 4})])
def test_latent_attention_alone(tmp_path, mix):
    """One layer without a feed-forward: prompt, token by token, and portions, against the oracle's residual stream."""
    from mistral_inference_b200.registry import load_model

    cfg = make_config(width=32, vocab=16, layers=[(mix, None)])
    w = make_weights(cfg, 1)
    m = load_model(write_folder(tmp_path / "m", cfg, w), device=DEV, dtype=torch.float32)
    toks = _tokens(cfg, 45, 3)
    taps = []
    O.forward(cfg, w, toks, taps)
    for portions in (None, [1] * 45, [20, 2, 23], [44, 1]):
        _close(_hidden(m, toks, portions), taps[0], torch.float32, str(portions))


@pytest.mark.parametrize("sizes", [dict(dim=32, rot_dim=32, vdim=32), dict(dim=64, rot_dim=32, vdim=64), dict(dim=16, rot_dim=16, vdim=32),
                                   dict(dim=128, rot_dim=64, vdim=128)])
def test_whole_prompts_on_the_tensor_cores(tmp_path, sizes):
    """bf16 prompts of head sizes that the tensor-core kernel takes run as multi-head attention over written-out keys and values;
    the result must agree with the latent form (same model, switch off) and with the oracle, also in a ragged batch, and decoding
    continues from the latent ring that the prompt left."""
    from mistral_inference_b200.registry import load_model

    mix = mixer_cfg(heads=3, q_rank=24, kv_rank=48, rot={"base": 1000.0, "dims": sizes["rot_dim"]}, **sizes)
    cfg = make_config(width=64, vocab=40, layers=[(mix, moe_cfg()), (mix, None)])
    w = {k: v.to(torch.bfloat16) for k, v in make_weights(cfg, 2).items()}
    m = load_model(write_folder(tmp_path / "m", cfg, w), device=DEV, dtype=torch.bfloat16)
    lens = [70, 16, 130]
    reqs = [_tokens(cfg, n + 3, 30 + i) for i, n in enumerate(lens)]
    refs = [O.forward(cfg, f32(w), r) for r in reqs]
    outs = {}
    for on in (True, False):
        for blk in m.layers:
            blk.mix.expand_prompts = on
        cache = m.make_cache(3, 140)
        got = m.forward(torch.tensor([t for r, n in zip(reqs, lens) for t in r[:n]], device=DEV), lens, cache)
        o, per = 0, []
        for n in lens:
            per.append([got[o:o + n]])
            o += n
        for k in range(3):
            step = m.forward(torch.tensor([r[n + k] for r, n in zip(reqs, lens)], device=DEV), [1, 1, 1], cache)
            for i in range(3):
                per[i].append(step[i:i + 1])
        outs[on] = [torch.cat(p) for p in per]
        for i in range(3):
            _close(outs[on][i], refs[i], torch.bfloat16, f"expanded={on} request {i}")
    if (sizes["dim"] + sizes["rot_dim"], sizes["vdim"]) in __import__("mistral_inference_b200._abi_hybrid", fromlist=["x"]).FLASH_SIZES:
        assert not torch.equal(outs[True][2], outs[False][2]), "the switch changed nothing: the tensor-core path did not run"


# ----------------------------------------------------------------------------- whole models through the cache
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(SHAPES))
def test_whole_prompt_matches_the_oracle(tmp_path, name, dtype):
    m, cfg, w = _model(tmp_path, name, dtype)
    toks = _tokens(cfg, 70, 1)
    ref = O.forward(cfg, w, toks)
    _close(m.forward(torch.tensor(toks, device=DEV), [len(toks)], None), ref, dtype)


def test_every_layer_run_matches(tmp_path):
    m, cfg, w = _model(tmp_path, "odd", torch.float32)
    toks = _tokens(cfg, 19, 4)
    taps, got = [], []
    O.forward(cfg, w, toks, taps)
    m._tap = lambda r, x: got.append(x.clone())
    try:
        m.forward(torch.tensor(toks, device=DEV), [len(toks)], None)
    finally:
        m._tap = None
    assert len(got) == len(taps) == 8    # layers 1 and 2 run three times
    for r, (a, b) in enumerate(zip(got, taps)):
        _close(a, b, torch.float32, f"layer run {r}")


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
    rows (with the earlier keys still in memory) and must not see them."""
    m, cfg, w = _model(tmp_path, "odd", dtype)
    lens, starts = [9, 30, 17], [5, 22, 1]
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
        rows = {i: [] for i in live}
        for i in live:
            rows[i].append(out[o:o + at[i]].clone())
            o += at[i]
        while live:
            gone = [k for k, i in enumerate(live) if at[i] == lens[i]]
            if gone:
                cache.retire(gone)
                live = [i for k, i in enumerate(live) if k not in gone]
                continue
            out = m.forward(torch.tensor([reqs[i][at[i]] for i in live], device=DEV), [1] * len(live), cache)
            for k, i in enumerate(live):
                rows[i].append(out[k:k + 1].clone())
                at[i] += 1
        for i in rows:
            _close(torch.cat(rows[i]), refs[i], dtype, f"round {round_} request {i}")
        reqs = reqs[::-1]; refs = refs[::-1]; lens = lens[::-1]; starts = [3, 8, 2]


def test_far_keys_and_long_decoding(tmp_path):
    """A sharp softmax (large scale) over 700 positions: a key that is lost, or taken from the wrong ring row, moves the result by
    far more than the tolerance.  The prompt ends inside the attention kernel's second round of key chunks, decoding crosses it."""
    sharp = mixer_cfg(heads=2, dim=16, rot_dim=8, vdim=16, q_rank=24, kv_rank=24, scale=1.2, rot={"base": 3000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    m, cfg, w = _model(tmp_path, "odd", torch.float32, layers=[(sharp, moe_cfg()), (sharp, None)], loop=(0, 1, 2))
    toks = _tokens(cfg, 700, 7)
    ref = O.forward(cfg, w, toks)
    cache = m.make_cache(1, 700)
    out = [m.forward(torch.tensor(toks[:500], device=DEV), [500], cache)]
    for t in toks[500:]:
        out.append(m.forward(torch.tensor([t], device=DEV), [1], cache))
    _close(torch.cat(out), ref, torch.float32)
    for blk in m.layers:   # the per-head decode kernel must give the same
        blk.mix.shared_decode = False
    cache = m.make_cache(1, 700)
    out = [m.forward(torch.tensor(toks[:640], device=DEV), [640], cache)]
    for t in toks[640:]:
        out.append(m.forward(torch.tensor([t], device=DEV), [1], cache))
    _close(torch.cat(out), ref, torch.float32, "per-head decode kernel")
    for blk in m.layers:
        blk.mix.shared_decode = True
    # the same, in one batch with a short request: the long one's keys are split over several CTAs
    cache = m.make_cache(2, 700)
    both = m.forward(torch.tensor(toks + toks[:3], device=DEV), [700, 3], cache)
    _close(both[:700], ref, torch.float32, "long request of a batch")
    _close(both[700:], ref[:3], torch.float32, "short request of a batch")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_generate(tmp_path, dtype):
    from mistral_inference_b200.generate import generate

    m, cfg, w = _model(tmp_path, "single", dtype)
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


def test_generate_command_line(tmp_path, capsys):
    from mistral_inference_b200.main import main

    cfg = make_config(**SHAPES["single"])
    w = make_weights(cfg, 4)
    folder = write_folder(tmp_path / "cli", cfg, w)
    assert main(["generate", str(folder), "--prompt", "5 17 3", "--prompt", "1 2", "--max-tokens", "4", "--dtype", "float32"]) == 0
    rows = [[int(t) for t in line.split()] for line in capsys.readouterr().out.strip().splitlines()]
    assert len(rows) == 2 and all(len(r) == 4 for r in rows)
    for prompt, got in zip(([5, 17, 3], [1, 2]), rows):
        seq = list(prompt)
        for tok in got:
            assert tok == int(O.forward(cfg, w, seq)[-1].argmax())
            seq.append(tok)
