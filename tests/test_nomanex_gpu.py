"""Nomanex through the engine against the plain oracle (oracle/nomanex_oracle.py): each mechanism alone, prefill against
token-by-token decoding, portions down to two tokens, unequal batches, pages and slots used again, window edges and far
keys made visible by construction, other sizes (also the degenerate ones), long decoding, and greedy generation through
the engine's own submit / scheduler / sampling path.  Configurations and weights are made here; nothing is read from disk
but what the test wrote."""
import numpy as np
import pytest

from nomanex_util import (dense, feed_portions, feed_whole, gla, latent, make_config, moe, open_engine, oracle_for, random_weights,
                          rel_err, write_model_dir)

pytestmark = pytest.mark.gpu

F32_TOL = 2e-5     # fp32 engine vs float64 oracle, relative RMS over the vocabulary


def close32(got, want, scale=1.0):
    """fp32 engine against the float64 oracle.  Nearly every row agrees to a few 1e-6; a row whose recurrent output is
    normalised from a nearly cancelled sum is legitimately worse conditioned, so the bound on the worst row is looser
    than the bound on the typical one."""
    r = rel_err(got, want)
    assert np.median(r) < F32_TOL * scale, np.median(r)
    assert r.max() < 15 * F32_TOL * scale, (int(np.argmax(r)), r.max())


def close16(got, want):
    """bf16 serving precision on these tiny widths: a few percent per row; a row where rounding flips a close routing
    choice may be far off, so the bound is on the median and on the 90th percentile."""
    r = rel_err(got, want)
    assert np.median(r) < 0.06, np.median(r)
    assert np.quantile(r, 0.9) < 0.2, np.quantile(r, 0.9)


def toks(n, vocab, seed=0):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def build(tmp_path, layers, seed=0, a_rank=4, q_gain=1.0, **kw):
    cfg = make_config(layers, **kw)
    W = random_weights(cfg, seed=seed, a_rank=a_rank, q_gain=q_gain)
    return cfg, W, write_model_dir(tmp_path / "m", cfg, W)


MIX = [(latent(), dense()), (gla(), moe()), (gla(heads=3, dim=8, vdim=4), None), ("weights_of", 1), (latent(window=9), moe(top=1)),
       ("weights_of", 0)]


@pytest.fixture(scope="module")
def mix(tmp_path_factory):
    cfg, W, d = build(tmp_path_factory.mktemp("mix"), MIX)
    return cfg, W, d, oracle_for(cfg, W)


@pytest.fixture(scope="module")
def mix_wide(tmp_path_factory):
    """The same stack with one window longer than any test sequence: no page falls behind every window, so a sequence
    holds all its pages and a small pool really fills."""
    layers = [(latent(window=500), dense())] + MIX[1:]
    cfg, W, d = build(tmp_path_factory.mktemp("mixw"), layers, seed=5)
    return cfg, W, d, oracle_for(cfg, W)


# ---------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("name,layers", [
    ("gla", [(gla(), None)]),
    ("gla_wide_value", [(gla(heads=1, dim=4, vdim=20), None)]),
    ("gla_many_rows", [(gla(heads=2, dim=40, vdim=8), None)]),       # more key rows than one thread holds: two row slices
    ("latent", [(latent(), None)]),
    ("latent_partial_rotation", [(latent(rot_dim=8, rot_dims=4), None)]),
    ("latent_one_head", [(latent(heads=1, dim=4, rot_dim=2, vdim=6, kv_rank=5, window=3), None)]),
    ("dense", [(gla(), dense())]),
    ("moe", [(gla(), moe())]),
    ("moe_one_group", [(gla(), moe(experts=5, top=3, count=1, keep=1))]),
    ("moe_all_groups_top1", [(latent(), moe(experts=8, top=1, count=4, keep=4))]),
    ("shared_weights", [(gla(), dense()), ("weights_of", 0), ("weights_of", 1)]),
])
def test_each_mechanism_matches_the_oracle(tmp_path, name, layers):
    cfg, W, d = build(tmp_path, layers, seed=3)
    o = oracle_for(cfg, W)
    t = toks(29, cfg["vocab"], 1)
    want, layers_want = o.forward(t, return_layers=True)
    with open_engine(d) as e:
        e.debug_residuals(True)
        got = feed_whole(e, t)
        res = e.read_residuals().reshape(layers_want.shape)
    assert np.abs(res - layers_want).max() < 1e-4 * max(1.0, np.abs(layers_want).max()), name
    close32(got, want)


def test_bfloat16_serving_precision_stays_near_the_oracle(mix):
    cfg, W, d, o = mix
    t = toks(70, cfg["vocab"], 2)
    want = o.forward(t)
    with open_engine(d, dtype="bfloat16") as e:
        got = feed_whole(e, t)
        dec = feed_portions(e, t, [40, 1])
    close16(got, want)
    close16(dec, want)


def test_bfloat16_widths_the_tensor_core_projection_cannot_take(tmp_path):
    """width and inner sizes that are no multiple of 8 run on the general linear kernels."""
    cfg, W, d = build(tmp_path, [(latent(kv_rank=11, vdim=6), dense(ff=13)), (gla(dim=6, vdim=10), moe(ff=7))], width=20, vocab=33)
    t = toks(40, 33, 4)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d, dtype="bfloat16") as e:
        close16(feed_whole(e, t), want)
    with open_engine(d) as e:
        close32(feed_whole(e, t), want)


@pytest.mark.parametrize("heads,kv_rank,rot_dim,window", [(2, 16, 16, 100), (16, 48, 16, 70), (20, 32, 32, 33), (3, 16, 16, 500)])
def test_bfloat16_tensor_core_attention_equals_the_plain_kernel(tmp_path, monkeypatch, heads, kv_rank, rot_dim, window):
    """Latent widths that fit the mma fragments take the tensor-core attention kernel: several 64-key tiles per window,
    several tokens per 16-row tile (few heads), several head groups (more than 16 heads), portions and decoding."""
    layers = [(latent(heads=heads, dim=8, rot_dim=rot_dim, vdim=8, kv_rank=kv_rank, window=window), None)]
    cfg, W, d = build(tmp_path, layers, seed=21, q_gain=3.0, width=32)
    t = toks(230, cfg["vocab"], 22)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d, dtype="bfloat16") as e:
        whole = feed_whole(e, t)
        cut = feed_portions(e, t, [67, 2, 90, 1])
    monkeypatch.setenv("B200_NX_ATTN_MMA", "0")
    with open_engine(d, dtype="bfloat16") as e:
        plain = feed_whole(e, t)
    monkeypatch.delenv("B200_NX_ATTN_MMA")
    monkeypatch.setenv("B200_NX_ATTN_SPLIT", "3")      # every window cut over three CTAs and merged
    with open_engine(d, dtype="bfloat16") as e:
        split = feed_portions(e, t, [67, 2, 90, 1])
    monkeypatch.delenv("B200_NX_ATTN_SPLIT")
    monkeypatch.setenv("B200_NX_ATTN_WIDE", "1")       # the 64-row kernel of large prompt steps, forced on this small one
    with open_engine(d, dtype="bfloat16") as e:
        wide = feed_whole(e, t)
        wide_cut = feed_portions(e, t, [67, 2, 90, 1])
    close16(whole, want)
    close16(cut, want)
    close16(split, want)
    close16(wide, want)
    close16(wide_cut, want)
    assert np.median(rel_err(wide, plain)) < 0.02 and np.median(rel_err(wide_cut, plain)) < 0.02
    assert rel_err(wide, plain).max() < 0.1 and rel_err(wide_cut, plain).max() < 0.1
    assert np.median(rel_err(whole, plain)) < 0.02 and np.median(rel_err(cut, plain)) < 0.02
    assert rel_err(whole, plain).max() < 0.1 and rel_err(cut, plain).max() < 0.1
    assert np.median(rel_err(split, cut)) < 0.02 and rel_err(split, cut).max() < 0.1


def test_bfloat16_large_prompt_step_takes_the_64_row_attention_kernel_by_itself(tmp_path, monkeypatch):
    """A step with query tiles enough for every SM (two prompts of 330 tokens, 16 heads: 4 tokens per 64-row tile) is
    dispatched to the 64-row kernel without any knob; it must agree with the oracle and with the plain kernel, windows
    crossing several 32-key tiles and both prompts' first tokens included."""
    layers = [(latent(heads=16, dim=8, rot_dim=16, vdim=8, kv_rank=48, window=75), None)]
    cfg, W, d = build(tmp_path, layers, seed=23, q_gain=3.0, width=32)
    seqs = [toks(330, cfg["vocab"], 24 + i) for i in range(2)]
    o = oracle_for(cfg, W)
    want = np.concatenate([o.forward(t) for t in seqs])

    def both(e):
        rids = [e.feed_open() for _ in seqs]
        out = e.feed_step([(r, t, list(range(len(t)))) for r, t in zip(rids, seqs)])
        for r in rids:
            e.feed_close(r)
        return out

    with open_engine(d, dtype="bfloat16", max_tokens=1024, max_seqs=2) as e:
        got = both(e)
    monkeypatch.setenv("B200_NX_ATTN_MMA", "0")
    with open_engine(d, dtype="bfloat16", max_tokens=1024, max_seqs=2) as e:
        plain = both(e)
    close16(got, want)
    assert np.median(rel_err(got, plain)) < 0.02 and rel_err(got, plain).max() < 0.1


def test_bfloat16_per_expert_tensor_core_path_equals_the_grouped_kernel(tmp_path, monkeypatch):
    """Large steps run every expert's rows as one tensor-core GEMM after reading the row counts back; forced here for
    small steps, including experts that get no token at all."""
    cfg, W, d = build(tmp_path, [(gla(), moe(experts=12, top=3, count=4, keep=2, ff=16)), (latent(), moe(experts=4, top=1, count=1, keep=1, ff=8))],
                      seed=31, width=32)
    t = toks(150, cfg["vocab"], 32)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d, dtype="bfloat16") as e:
        grouped = feed_whole(e, t)
    monkeypatch.setenv("B200_NX_MOE_TC_MIN_T", "1")
    with open_engine(d, dtype="bfloat16") as e:
        per_expert = feed_whole(e, t)
        cut = feed_portions(e, t, [3, 70, 1])
    close16(per_expert, want)
    close16(cut, want)
    assert np.median(rel_err(per_expert, grouped)) < 0.03


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_medium_odd_shapes_on_every_projection_path(tmp_path, dtype):
    """Sizes between the toy ones and a real layer, none of them round: projections wide enough for several tensor-core
    weight slabs, a latent width that fits the mma fragments (80) beside one that does not (72 + 4), experts whose hidden
    size is no multiple of 8 beside ones that are, steps above and below the per-expert threshold."""
    layers = [(latent(heads=5, dim=24, rot_dim=16, vdim=40, kv_rank=64, window=50), dense(ff=328, limit=3.0)),
              (gla(heads=3, dim=40, vdim=24, tau=12.0), moe(experts=10, top=3, count=5, keep=3, ff=72)),
              (latent(heads=6, dim=16, rot_dim=4, vdim=24, kv_rank=72, window=200), moe(experts=6, top=2, count=2, keep=1, ff=20)),
              ("weights_of", 1), (gla(heads=7, dim=8, vdim=16, tau=4.0), None)]
    cfg, W, d = build(tmp_path, layers, seed=41, a_rank=12, width=200, vocab=301, buckets=997, mul_prev=131, mul_cur=31)
    t = toks(300, cfg["vocab"], 42)
    want = oracle_for(cfg, W).forward(t)
    close = close16 if dtype == "bfloat16" else close32
    with open_engine(d, dtype=dtype) as e:
        close(feed_whole(e, t), want)
        close(feed_portions(e, t, [130, 3, 150, 1]), want)


# ---------------------------------------------------------------- prefill, decoding, portions
def test_prefill_equals_token_by_token_decoding(mix):
    cfg, W, d, o = mix
    t = toks(45, cfg["vocab"], 16)
    want = o.forward(t)
    with open_engine(d) as e:
        whole = feed_whole(e, t)
        single = feed_portions(e, t, [1])
    close32(whole, want)
    close32(single, want)
    assert np.abs(whole - single).max() < 1e-4


@pytest.mark.parametrize("sizes", [[2], [3, 2, 7, 1, 1, 16, 5], [17, 2, 2, 31], [64, 1], [5, 70, 2, 1]])
def test_portions_of_any_size_give_the_same_logits(mix, sizes):
    cfg, W, d, o = mix
    t = toks(97, cfg["vocab"], 6)
    want = o.forward(t)
    with open_engine(d) as e:
        got = feed_portions(e, t, sizes)
    close32(got, want)


def test_long_decoding_stays_on_the_oracle(tmp_path):
    cfg, W, d = build(tmp_path, [(latent(window=20), None), (gla(tau=30.0), dense())], seed=8)
    t = toks(260, cfg["vocab"], 7)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d) as e:
        got = feed_portions(e, t, [20, 1])
    close32(got, want, 5)


# ---------------------------------------------------------------- batches, pages, slots
def test_unequal_requests_in_one_batch_equal_each_alone(mix):
    cfg, W, d, o = mix
    seqs = [toks(n, cfg["vocab"], 10 + i) for i, n in enumerate((50, 23, 9, 77))]
    want = [o.forward(t) for t in seqs]
    with open_engine(d, max_tokens=128) as e:
        rids = [e.feed_open() for _ in seqs]
        at = [0] * 4
        got = [[] for _ in seqs]
        plan = [(7, 1, 9, 30), (20, 1, 0, 2), (1, 3, 0, 17), (22, 1, 0, 1), (0, 17, 0, 27)]
        step = 0
        while any(at[i] < len(seqs[i]) for i in range(4)):
            entries, idx = [], []
            for i in range(4):
                n = min(plan[min(step, len(plan) - 1)][i] or (1 if step >= len(plan) else 0), len(seqs[i]) - at[i])
                if n > 0:
                    entries.append((rids[i], seqs[i][at[i]:at[i] + n], list(range(n))))
                    idx.append((i, n))
            out = e.feed_step(entries)
            r = 0
            for i, n in idx:
                got[i].append(out[r:r + n])
                at[i] += n
                r += n
            step += 1
        for r in rids:
            e.feed_close(r)
    for i in range(4):
        close32(np.concatenate(got[i]), want[i])


def test_pages_and_slots_are_used_again(mix):
    """A pool of exactly two sequences' pages and two slots: later requests run in what earlier ones gave back."""
    cfg, W, d, o = mix
    seqs = [toks(n, cfg["vocab"], 20 + i) for i, n in enumerate((40, 33, 48, 17, 41))]
    with open_engine(d, max_tokens=48, max_seqs=2, blocks=6, budget=96) as e:
        a, b = e.feed_open(), e.feed_open()
        e.feed_step([(a, seqs[0], []), (b, seqs[1][:20], [])])
        e.feed_step([(b, seqs[1][20:], [])])
        e.feed_close(a)
        c = e.feed_open()                      # takes a's slot and pages while b is still live
        got_c = e.feed_step([(c, seqs[2][:30], list(range(30)))])
        e.feed_close(b)
        f = e.feed_open()
        out = e.feed_step([(c, seqs[2][30:], list(range(18))), (f, seqs[3], list(range(17)))])
        got_c = np.concatenate([got_c, out[:18]])
        got_f = out[18:]
        e.feed_close(c)
        e.feed_close(f)
        g = e.feed_open()
        got_g = feed_portions_on(e, g, seqs[4], [16, 1])
        assert e.stats().kv_blocks_free == 6
    close32(got_c, o.forward(seqs[2]))
    close32(got_f, o.forward(seqs[3]))
    close32(got_g, o.forward(seqs[4]))


def feed_portions_on(e, r, tokens, sizes):
    outs, at, i = [], 0, 0
    while at < len(tokens):
        n = min(sizes[min(i, len(sizes) - 1)], len(tokens) - at)
        outs.append(e.feed_step([(r, tokens[at:at + n], list(range(n)))]))
        at += n
        i += 1
    e.feed_close(r)
    return np.concatenate(outs)


def test_pages_behind_every_window_go_back_to_the_pool_while_the_sequence_runs(tmp_path):
    """Two 380-token sequences side by side in a pool that could not hold both whole (30 pages of 16 tokens for 2 x 24):
    pages that no layer's window reaches any more are returned as the sequences advance, and the logits do not change."""
    cfg, W, d = build(tmp_path, [(latent(window=20), dense()), (gla(), None), (latent(window=33, kv_rank=16, rot_dim=16), None)], seed=61)
    o = oracle_for(cfg, W)
    seqs = [toks(380, cfg["vocab"], 62 + i) for i in range(2)]
    want = [o.forward(t) for t in seqs]
    with open_engine(d, max_tokens=400, max_seqs=2, blocks=30, budget=64) as e:
        rids = [e.feed_open() for _ in seqs]
        got = [[], []]
        at = 0
        sizes = [16, 7, 16, 1, 2, 16]
        i = 0
        while at < 380:
            n = min(sizes[i % len(sizes)], 380 - at)
            out = e.feed_step([(r, t[at:at + n], list(range(n))) for r, t in zip(rids, seqs)])
            got[0].append(out[:n])
            got[1].append(out[n:])
            at += n
            i += 1
            assert e.stats().kv_blocks_free >= 30 - 2 * 5       # window 33 + a 16-token portion: at most 5 pages each
        for r in rids:
            e.feed_close(r)
        assert e.stats().kv_blocks_free == 30
    for k in range(2):
        close32(np.concatenate(got[k]), want[k], 3)


def test_a_step_over_the_pool_is_refused_and_leaves_the_engine_usable(mix_wide):
    from kubeai_b200 import B200Error
    cfg, W, d, o = mix_wide
    t = toks(40, cfg["vocab"], 30)
    with open_engine(d, max_tokens=48, max_seqs=2, blocks=3) as e:
        a, b = e.feed_open(), e.feed_open()
        e.feed_step([(a, t[:30], [])])
        with pytest.raises(B200Error):
            e.feed_step([(b, t[:30], [])])        # 2 + 2 pages do not fit 3
        e.feed_close(b)
        got = e.feed_step([(a, t[30:], list(range(10)))])
        e.feed_close(a)
    close32(got, o.forward(t)[30:])


# ---------------------------------------------------------------- windows, far keys, first tokens
@pytest.mark.parametrize("window", [1, 2, 16, 17, 33, 500])
def test_window_edge_is_exact_in_prompts_and_in_decoding(tmp_path, window):
    """Sharp queries make single keys matter: the oracle with a window one shorter or longer is far from the engine."""
    layers = [(latent(window=window, kv_rank=10), None)]
    cfg, W, d = build(tmp_path, layers, seed=11, q_gain=6.0)
    t = toks(60, cfg["vocab"], 12)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d) as e:
        whole = feed_whole(e, t)
        dec = feed_portions(e, t, [window + 3, 1]) if window < 50 else feed_portions(e, t, [7, 1])
        cut = feed_portions(e, t, [max(2, window - 1), 2, window + 1])
    for got in (whole, dec, cut):
        close32(got, want, 2)
    for other in (window - 1, window + 1):
        if other < 1 or window >= 60:
            continue
        cfg2 = make_config([(latent(window=other, kv_rank=10), None)])
        off = rel_err(oracle_for(cfg2, W).forward(t), want)
        assert off.max() > 100 * F32_TOL, "the test's weights do not show the window edge"


def test_far_tokens_reach_through_the_recurrent_state(tmp_path):
    """Slow decay (large tau, large bias): a token hundreds of positions back still moves the logits, in prompt portions
    and in decoding alike; changing only that token changes the last logits."""
    cfg, W, d = build(tmp_path, [(gla(tau=200.0), None)], seed=13)
    W["l0.mix.a2.b"] = W["l0.mix.a2.b"] + 6.0
    d = write_model_dir(tmp_path / "far", cfg, W)
    o = oracle_for(cfg, W)
    t = toks(300, cfg["vocab"], 14)
    t2 = list(t)
    t2[3] = (t[3] + 1) % cfg["vocab"]
    want, want2 = o.forward(t), o.forward(t2)
    assert rel_err(want2[-1:], want[-1:]).max() > 100 * F32_TOL, "the test's weights do not show the far token"
    with open_engine(d) as e:
        got = feed_portions(e, t, [130, 2, 120, 1])
        whole = feed_whole(e, t)
        got2 = feed_portions(e, t2, [64])
    # a decay this close to 1 is itself rounded in fp32, and 300 such steps multiply: looser against the float64 oracle,
    # tight between the engine's own ways of cutting the same sequence
    close32(got, want, 10)
    close32(got2, want2, 10)
    assert np.abs(got - whole).max() < 1e-4


def test_first_tokens_and_the_bigram_rows(mix):
    cfg, W, d, o = mix
    with open_engine(d) as e:
        for t in ([5], [5, 5], [0, 39], [39, 0, 0, 1]):
            close32(feed_whole(e, t), o.forward(t))
            close32(feed_portions(e, t, [1]), o.forward(t))


# ---------------------------------------------------------------- other sizes
@pytest.mark.parametrize("seed", range(6))
def test_random_configurations(tmp_path, seed):
    rng = np.random.default_rng(100 + seed)
    layers = []
    for i in range(int(rng.integers(1, 5))):
        if i > 0 and rng.random() < 0.3:
            layers.append(("weights_of", int(rng.integers(0, i))))
            if layers[layers[-1][1]][0] == "weights_of":
                layers[-1] = ("weights_of", layers[layers[-1][1]][1])
            continue
        if rng.random() < 0.5:
            mixer = gla(heads=int(rng.integers(1, 4)), dim=int(rng.integers(1, 13)), vdim=int(rng.integers(1, 13)), tau=float(rng.uniform(1, 40)))
        else:
            rd = 2 * int(rng.integers(1, 4))
            mixer = latent(heads=int(rng.integers(1, 4)), dim=int(rng.integers(1, 10)), rot_dim=rd, rot_dims=2 * int(rng.integers(1, rd // 2 + 1)),
                           vdim=int(rng.integers(1, 10)), kv_rank=int(rng.integers(2, 20)), window=int(rng.integers(1, 40)),
                           base=float(rng.uniform(10, 1e5)), scale=float(rng.uniform(0.1, 0.6)))
        r = rng.random()
        if r < 0.3:
            mlp = None
        elif r < 0.6:
            mlp = dense(ff=int(rng.integers(1, 30)), limit=float(rng.uniform(0.5, 4)))
        else:
            count = int(rng.integers(1, 4))
            per = int(rng.integers(1, 4))
            keep = int(rng.integers(1, count + 1))
            mlp = moe(experts=count * per, top=int(rng.integers(1, keep * per + 1)), count=count, keep=keep, ff=int(rng.integers(1, 12)))
        layers.append((mixer, mlp))
    cfg, W, d = build(tmp_path, layers, seed=seed, a_rank=int(rng.integers(1, 7)), width=int(rng.integers(3, 40)), vocab=int(rng.integers(2, 60)),
                      buckets=int(rng.integers(1, 30)), mul_prev=int(rng.integers(0, 1000)), mul_cur=int(rng.integers(0, 1000)),
                      mult=float(rng.uniform(0.2, 1.0)), eps=float(10 ** rng.uniform(-6, -3)))
    t = toks(50, cfg["vocab"], seed)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d) as e:
        close32(feed_whole(e, t), want, 2)
        close32(feed_portions(e, t, [9, 2, 1]), want, 2)


# ---------------------------------------------------------------- the engine's own entry point
def greedy_agrees(o, prompt, got):
    """Compare token by token while the oracle's own top-2 margin is clear."""
    seq = list(prompt)
    for g in got:
        row = np.sort(o.forward(seq)[-1])
        w = int(np.argmax(o.forward(seq)[-1]))
        if row[-1] - row[-2] < 1e-3:
            return
        assert g == w, (len(seq) - len(prompt), g, w)
        seq.append(g)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_submit_scheduler_and_sampler(mix, dtype):
    """More requests than slots, a token budget that cuts prompts into portions, generation by the engine's argmax."""
    cfg, W, d, o = mix
    prompts = [toks(n, cfg["vocab"], 40 + i) for i, n in enumerate((37, 5, 21, 50, 2))]
    with open_engine(d, dtype=dtype, max_tokens=96, max_seqs=2, budget=16, blocks=12) as e:
        outs = e.generate(prompts, max_tokens=12)
        st = e.stats()
    assert st.kv_blocks_free == 12
    for p, got in zip(prompts, outs):
        assert len(got) == 12
        if dtype == "float32":
            greedy_agrees(o, p, got)
    if dtype == "bfloat16":
        # bf16 rounding may flip a close call; the first token of every request must still be the oracle's unless it is one
        for p, got in zip(prompts, outs):
            row = np.sort(o.forward(p)[-1])
            if row[-1] - row[-2] > 0.3:
                assert got[0] == int(np.argmax(o.forward(p)[-1]))


def test_preemption_recomputes_state_from_the_start(mix_wide):
    """A pool too small for all running sequences to finish: the scheduler preempts and recomputes; outputs do not change."""
    cfg, W, d, o = mix_wide
    prompts = [toks(n, cfg["vocab"], 60 + i) for i, n in enumerate((30, 28, 31))]
    with open_engine(d, max_tokens=64, max_seqs=3, budget=64, blocks=8) as e:
        outs = e.generate(prompts, max_tokens=20)
        assert e.stats().preemptions > 0
    for p, got in zip(prompts, outs):
        greedy_agrees(o, p, got)


def test_chat_completion_through_the_serving_shell(tmp_path):
    """The design behind the HTTP handler chain, stepped by the engine's own background loop: prompt rendering, submit,
    continuous batching of two concurrent requests, greedy sampling, SSE framing; the tokens are the oracle's."""
    import json
    import threading
    from kubeai_b200.engine import Engine, default_config
    from kubeai_b200.server import Server, tokenize
    V = 300
    cfg, W, d = build(tmp_path, MIX, seed=51, vocab=V)
    o = oracle_for(cfg, W)
    lim = default_config(manual_step=0, enable_prefix_caching=0, max_num_seqs=4, max_batched_tokens=32, max_model_len=256, num_kv_blocks=64)
    eng = Engine(lim, d, dtype="float32")
    srv = Server([eng], model="nx", vocab=V, max_model_len=256)
    try:
        out = {}

        def ask(i, text):
            body = dict(model="nx", messages=[{"role": "user", "content": text}], max_tokens=5, temperature=0, stream=(i == 0))
            out[i] = srv.handle("POST", "/openai/v1/chat/completions", json.dumps(body))

        th = [threading.Thread(target=ask, args=(i, t)) for i, t in enumerate(["Hello there, how are you?", "Hi"])]
        for t in th:
            t.start()
        for t in th:
            t.join()
        assert out[0].status == 200 and out[1].status == 200
        ev = out[0].sse_events()
        assert ev[-1] == "[DONE]"
        text0 = "".join(json.loads(e)["choices"][0]["delta"].get("content", "") for e in ev[:-1] if json.loads(e)["choices"])
        text1 = out[1].json()["choices"][0]["message"]["content"]
        for text, user in ((text0, "Hello there, how are you?"), (text1, "Hi")):
            prompt = srv.render_prompt("/v1/chat/completions", json.dumps(dict(model="nx", messages=[{"role": "user", "content": user}])))
            got = tokenize(text, V)
            assert len(got) == 5
            greedy_agrees(o, prompt, got)
    finally:
        srv.close()
        eng.close()


def test_unknown_architecture_and_bad_config_are_refused(tmp_path):
    from kubeai_b200 import B200Error
    cfg, W, d = build(tmp_path, [(gla(), None)])
    bad = dict(cfg, architecture="Nomanex2")
    with pytest.raises(B200Error, match="not registered"):
        open_engine(write_model_dir(tmp_path / "bad", bad, W))
    cyc = make_config([(gla(), None), (gla(), None)])
    cyc["layers"][0]["weights_of"] = 1
    cyc["layers"][1]["weights_of"] = 0
    with pytest.raises(B200Error, match="cycle"):
        open_engine(write_model_dir(tmp_path / "cyc", cyc, W))
    del W["l0.mix.k"]
    with pytest.raises(B200Error, match="l0.mix.k"):
        open_engine(write_model_dir(tmp_path / "missing", cfg, W))
