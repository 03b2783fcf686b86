"""The Zurevik design of the hybrid family on the GPU against the slow float64 oracle (tests/zurevik_oracle.py): each mechanism alone, and —
through Engine.trace_step, which drives the scheduler's own batch builder, pages and slots — prompts cut into portions, token-by-token
decoding, mixed batches, reused pages, window and kept-token edges in prompts and in decoding, and greedy generation through the scheduler.
Small random checkpoints are written per test; sharp queries make single keys decide so that a window that is one token off shows."""
import numpy as np
import pytest

import zurevik_oracle as Z

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4          # fp32 engine against the float64 oracle (relative to the logits' spread)
BF16_TOL = 0.12         # bf16 matrices / activations: worst row; the median is held to a quarter of it (a rounding may flip a near-tie expert choice)
SAME_TOL = 1e-5         # fp32 engine, two schedules: a row's arithmetic does not depend on how its prompt was cut or on its batch


def engine(folder, dtype="float32", pages=8, slots=4, **kw):
    from opsagent_b200 import Engine
    return Engine(dict({"model_dir": str(folder), "dtype": dtype, "num_pages": pages, "max_seq_len": 64 * pages, "max_step_tokens": 64 * pages,
                        "max_batch": slots, "prefix_cache": 0}, **kw))


def checkpoint(tmp_path, cfg, seed=0, **kw):
    W = Z.random_weights(cfg, seed, **kw)
    Z.write_checkpoint(str(tmp_path), cfg, W)
    return W


def tokens_of(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def replay(eng, rid, toks, cuts):
    """feed toks to request rid in portions of the given sizes (the rest one by one), wanting every position; -> logits [len(toks), vocab]"""
    out, at = [], 0
    sizes = list(cuts)
    while at < len(toks):
        n = min(sizes.pop(0) if sizes else 1, len(toks) - at)
        out.append(eng.trace_step([(rid, toks[at:at + n], list(range(n)))], [rid] if at + n == len(toks) else []))
        at += n
    return np.concatenate(out)


def check(got, want, dtype):
    e = Z.rel_err(got.astype(np.float64), want)
    if dtype == "float32":
        assert e.max() < F32_TOL, f"worst row {e.argmax()} differs by {e.max():.3e}"
    else:
        assert np.quantile(e, 0.9) < BF16_TOL and np.median(e) < BF16_TOL / 4, f"bf16 rows differ: median {np.median(e):.3e}, 90% {np.quantile(e, 0.9):.3e}"


MOE = Z.moe()
SINGLE = {
    "differential": [Z.diff_layer()],
    "differential_equal_heads_no_kept_tokens": [Z.diff_layer(heads=3, kv_heads=3, dim=12, vdim=10, window=9, keep_first=0, diff=0.7)],
    "differential_one_kv_head_window_beyond_prompt": [Z.diff_layer(heads=4, kv_heads=1, dim=16, vdim=32, window=500, keep_first=5, diff=0.1)],
    "sink": [Z.sink_layer()],
    "sink_window_of_one": [Z.sink_layer(heads=2, kv_heads=2, dim=8, vdim=12, window=1)],
    "sink_reading_an_earlier_cache": [Z.sink_layer(window=12), Z.diff_layer(), Z.sink_layer(window=40, kv_from=0)],
    "experts": [Z.sink_layer(mlp=MOE)],
    "experts_top1": [Z.diff_layer(mlp=Z.moe(experts=3, top=1, ff=10))],
    "experts_all_chosen": [Z.diff_layer(mlp=Z.moe(experts=4, top=4, ff=40))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = Z.make_config(SINGLE[name], width=40, vocab=77, embed_scale=1.5, softcap=0 if "sink" in name else 9.0)
    W = checkpoint(tmp_path, cfg, seed=len(name))
    toks = tokens_of(cfg, 70, 1)                       # crosses a page border
    want = Z.forward(cfg, W, toks)
    with engine(tmp_path, dtype) as eng:
        check(replay(eng, 1, toks, [70]), want, dtype)           # whole prompt
        check(replay(eng, 2, toks, [1, 1, 2, 3, 57, 2]), want, dtype)   # the first tokens alone, short portions, then token by token


def stack_cfg(**kw):
    layers = [Z.diff_layer(mlp=MOE), Z.sink_layer(window=37, mlp=MOE), Z.diff_layer(heads=2, kv_heads=1, dim=16, vdim=16, window=11, keep_first=2, diff=0.6, mlp=None),
              Z.sink_layer(window=70, kv_from=1, mlp=Z.moe(experts=5, top=3, ff=20)), Z.sink_layer(heads=2, kv_heads=1, dim=24, vdim=24, window=5, mlp=None)]
    return Z.make_config(layers, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_decoding_match_the_whole_prompt(tmp_path, dtype):
    cfg = stack_cfg()
    W = checkpoint(tmp_path, cfg, seed=3)
    toks = tokens_of(cfg, 140, 2)
    want = Z.forward(cfg, W, toks)
    with engine(tmp_path, dtype) as eng:
        outs = [replay(eng, 7, toks, cuts) for cuts in ([140], [2, 62, 1, 2, 61, 12], [63, 2, 64], [5], [127, 1, 1, 11], [64, 64, 2, 2, 2, 2, 2, 2])]
    for got in outs:
        check(got, want, dtype)
        if dtype == "float32":
            assert Z.rel_err(got.astype(np.float64), outs[0].astype(np.float64)).max() < SAME_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_and_reused_pages(tmp_path, dtype):
    """Requests at different stages share every step (a prompt portion beside single tokens); later requests take over the pages of finished
    ones: a stale cache row or a wrong block table would show.  Each request's rows equal the same request alone."""
    cfg = stack_cfg()
    W = checkpoint(tmp_path, cfg, seed=5)
    lens = {1: 100, 2: 37, 3: 66, 4: 90, 5: 20}
    toks = {r: tokens_of(cfg, n, 20 + r) for r, n in lens.items()}
    want = {r: Z.forward(cfg, W, toks[r]) for r in lens}
    got = {r: [] for r in lens}
    at = {r: 0 for r in lens}
    with engine(tmp_path, dtype, pages=4, slots=3) as eng:
        def step(parts):
            entries, end = [], []
            for r, n in parts:
                n = min(n, lens[r] - at[r])
                entries.append((r, toks[r][at[r]:at[r] + n], list(range(n))))
                at[r] += n
                if at[r] == lens[r]:
                    end.append(r)
            out = eng.trace_step(entries, end)
            k = 0
            for r, t, w in entries:
                got[r].append(out[k:k + len(w)])
                k += len(w)
        step([(1, 60)])
        step([(1, 1), (2, 30)])                       # 1 decodes beside a portion of 2
        step([(1, 3), (2, 7)])                        # 2 ends: its page is free
        step([(1, 36), (5, 2)])                       # 1 ends, 5 starts on 2's page
        step([(5, 18), (3, 64)])                      # 5 ends; 3 fills exactly one page
        step([(3, 2), (4, 2)])                        # 3 ends on a page's second token; 4 starts
        while at[4] < lens[4]:
            step([(4, 29)])
        assert eng.stats()["pages_free"] == 4
        for r in lens:                                # each alone, whole, in the same engine
            alone = replay(eng, 10 + r, toks[r], [lens[r]])
            assert Z.rel_err(np.concatenate(got[r]).astype(np.float64), alone.astype(np.float64)).max() < (SAME_TOL if dtype == "float32" else 2e-2)
    for r in lens:
        check(np.concatenate(got[r]), want[r], dtype)


def edge_cfg():
    # windows that end inside a page, on a page border (64) and beyond two pages; kept first tokens 1 and 6
    layers = [Z.diff_layer(heads=2, kv_heads=1, dim=16, vdim=16, window=50, keep_first=6, diff=0.4), Z.sink_layer(heads=2, kv_heads=2, dim=16, vdim=16, window=64),
              Z.diff_layer(heads=2, kv_heads=2, dim=8, vdim=16, window=130, keep_first=1, diff=0.2), Z.sink_layer(heads=2, kv_heads=2, dim=16, vdim=16, window=33, kv_from=1)]
    return Z.make_config(layers, width=48, vocab=64, softcap=15.0)


def test_window_and_kept_token_edges_decide_and_are_exact(tmp_path):
    """Sharp queries: single keys dominate each softmax, so a key just inside a window (or the last kept first token) carries real weight.
    The oracle itself shows it: a window one shorter, one kept token fewer or a dropped sink changes rows by far more than the tolerance.
    The engine must agree with the unchanged oracle in a whole prompt, in portions cut around the edges, and decoding over them."""
    cfg = edge_cfg()
    W = checkpoint(tmp_path, cfg, seed=8, sharp=6.0)
    toks = tokens_of(cfg, 300, 6)
    want = Z.forward(cfg, W, toks)

    def changed(fn):
        c = edge_cfg()
        fn(c["layers"])
        return Z.rel_err(Z.forward(c, W, toks), want)
    for li in range(4):
        shorter = changed(lambda L: L[li]["mixer"]["mask"].__setitem__("size", L[li]["mixer"]["mask"]["size"] - 1))
        longer = changed(lambda L: L[li]["mixer"]["mask"].__setitem__("size", L[li]["mixer"]["mask"]["size"] + 1))
        assert (shorter > 20 * F32_TOL).sum() > 10 and (longer > 20 * F32_TOL).sum() > 10, f"layer {li}: the window's edge does not show in the oracle"
    for li in (0, 2):
        fewer = changed(lambda L: L[li]["mixer"]["mask"].__setitem__("keep_first", L[li]["mixer"]["mask"]["keep_first"] - 1))
        more = changed(lambda L: L[li]["mixer"]["mask"].__setitem__("keep_first", L[li]["mixer"]["mask"]["keep_first"] + 1))
        assert (fewer > 20 * F32_TOL).sum() > 5 and (more > 20 * F32_TOL).sum() > 5, f"layer {li}: the kept tokens do not show in the oracle"
    no_sink = dict(W)
    no_sink["l1.mix.sink"] = np.full(2, -60.0)
    assert (Z.rel_err(Z.forward(cfg, no_sink, toks), want) > 20 * F32_TOL).sum() > 10
    with engine(tmp_path, pages=6) as eng:
        check(replay(eng, 1, toks, [300]), want, "float32")
        check(replay(eng, 2, toks, [49, 2, 13, 1, 63, 2, 2, 60, 4, 33]), want, "float32")      # portions that start and end around positions 50, 64, 130
        check(replay(eng, 3, toks, [40]), want, "float32")                                     # decodes over every edge and four page borders
    with engine(tmp_path, "bfloat16", pages=6) as eng:
        for cuts in ([300], [49, 2, 13, 1, 63, 2, 2, 60, 4, 33], [120]):
            e = Z.rel_err(replay(eng, 1, toks, cuts).astype(np.float64), want)
            assert np.quantile(e, 0.95) < 0.1 and e.max() < 0.35, f"bf16, cuts {cuts}: 95% {np.quantile(e, 0.95):.3e}, worst {e.max():.3e}"


def test_a_far_key_decides_through_pages_and_decoding(tmp_path):
    """A window of 400 over a 460-token prompt with sharp queries: keys hundreds of tokens back, on other pages, carry the answer (dropping the
    first page from the oracle's input changes the last rows), in a prompt and when decoding."""
    cfg = Z.make_config([Z.sink_layer(heads=2, kv_heads=1, dim=16, vdim=16, window=400), Z.diff_layer(heads=2, kv_heads=2, dim=16, vdim=16, window=400, keep_first=0, mlp=MOE)],
                        width=48, vocab=64)
    W = checkpoint(tmp_path, cfg, seed=9, sharp=6.0)
    toks = tokens_of(cfg, 460, 5)
    want = Z.forward(cfg, W, toks)
    assert Z.rel_err(Z.forward(cfg, W, toks[64:])[-40:], want[-40:]).max() > 50 * F32_TOL
    with engine(tmp_path, pages=8) as eng:
        check(replay(eng, 1, toks, [460]), want, "float32")
        check(replay(eng, 2, toks, [383, 2, 63]), want, "float32")       # decodes across the borders at 448 and while the window passes position 0 .. 60


def test_long_decoding(tmp_path):
    cfg = stack_cfg()
    W = checkpoint(tmp_path, cfg, seed=11)
    toks = tokens_of(cfg, 200, 7)
    with engine(tmp_path) as eng:
        check(replay(eng, 1, toks, [3]), Z.forward(cfg, W, toks), "float32")     # 197 single-token steps over three page borders, every window passed


TC_STACKS = {
    # head sizes that take the tensor-core attention kernels (dim a multiple of 16, vdim 16 / 32 / 64 / 96 / 128), windows that cut tiles
    "three_k_steps_and_96_value_channels": [Z.diff_layer(heads=4, kv_heads=2, dim=32, vdim=96, window=75, keep_first=5, diff=0.45, mlp=MOE),
                                            Z.sink_layer(heads=4, kv_heads=1, dim=48, vdim=32, window=141, mlp=Z.moe(experts=8, top=2, ff=64)),
                                            Z.diff_layer(heads=2, kv_heads=2, dim=16, vdim=16, window=200, keep_first=70, diff=0.25),
                                            Z.sink_layer(heads=2, kv_heads=1, dim=48, vdim=32, window=40, kv_from=1)],
    # the widest tiles (two maps x 128 value channels), a group of 8 heads per key/value head, and a group of 20: more query slots per decoding
    # row than the decoding form takes, so its rows go through the 64-slot form (no experts here: no choice can flip, the worst row stays sharp)
    "widest_tiles_and_large_groups": [Z.diff_layer(heads=2, kv_heads=1, dim=64, vdim=128, window=90, keep_first=33, diff=0.35),
                                      Z.sink_layer(heads=8, kv_heads=1, dim=128, vdim=64, window=65),
                                      Z.sink_layer(heads=40, kv_heads=2, dim=16, vdim=16, window=100),
                                      Z.diff_layer(heads=6, kv_heads=2, dim=16, vdim=64, window=31, keep_first=1, diff=0.8)],
}


@pytest.mark.parametrize("name", sorted(TC_STACKS))
def test_bf16_tensor_core_path_and_plain_path_agree_with_the_oracle(tmp_path, name):
    """Prompts long enough for several query and key tiles, whole, in portions that straddle tiles, and decoding (the split-key form), on the
    tensor-core kernels and on the plain kernels (hy_tensor_core = 0)."""
    cfg = Z.make_config(TC_STACKS[name], width=64, vocab=96)
    W = checkpoint(tmp_path, cfg, seed=13, sharp=2.0)
    toks = tokens_of(cfg, 330, 8)
    want = Z.forward(cfg, W, toks)
    for tc in (1, 0):
        with engine(tmp_path, "bfloat16", pages=6, hy_tensor_core=tc) as eng:
            for cuts in ([330], [17, 33, 63, 130, 41, 30], [300]):
                e = Z.rel_err(replay(eng, 1, toks, cuts).astype(np.float64), want)
                assert np.quantile(e, 0.95) < 0.08 and e.max() < 0.3, f"tensor cores {tc}, cuts {cuts}: 95% {np.quantile(e, 0.95):.3e}, worst {e.max():.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_fit_no_tile(tmp_path, dtype):
    """Widths and head sizes that are multiples of nothing: every product falls back to the plain GEMM and attention to the plain kernel."""
    layers = [Z.diff_layer(heads=3, kv_heads=1, dim=6, vdim=10, window=7, keep_first=9, diff=0.9, mlp=Z.moe(experts=3, top=2, ff=10)),
              Z.sink_layer(heads=6, kv_heads=3, dim=5, vdim=7, window=3, mlp=None), Z.sink_layer(heads=3, kv_heads=3, dim=5, vdim=7, window=90, kv_from=1, mlp=Z.moe(experts=7, top=3, ff=21))]
    cfg = Z.make_config(layers, width=36, vocab=51, embed_scale=0.5, softcap=4.0)
    W = checkpoint(tmp_path, cfg, seed=21)
    toks = tokens_of(cfg, 90, 11)
    want = Z.forward(cfg, W, toks)
    with engine(tmp_path, dtype) as eng:
        check(replay(eng, 1, toks, [90]), want, dtype)
        check(replay(eng, 2, toks, [2, 62, 3, 20]), want, dtype)


def test_router_bias_and_chosen_softmax_decide(tmp_path):
    """A router bias that dominates the logits picks the experts (the oracle without it answers differently), and the weights are the softmax
    over the chosen logits, not over all of them."""
    mlp = Z.moe(experts=8, top=3, ff=16)
    cfg = Z.make_config([Z.sink_layer(mlp=mlp), Z.diff_layer(mlp=mlp)], width=40, vocab=60)
    W = Z.random_weights(cfg, 23)
    rng = np.random.default_rng(5)
    for i in range(2):
        W["l%d.mlp.router.b" % i] = Z.bf16_round(3.0 * rng.standard_normal(8)).astype(np.float64)
    Z.write_checkpoint(str(tmp_path), cfg, W)
    toks = tokens_of(cfg, 70, 3)
    want = Z.forward(cfg, W, toks)
    plain = dict(W)
    for i in range(2):
        plain["l%d.mlp.router.b" % i] = np.zeros(8)
    assert Z.rel_err(Z.forward(cfg, plain, toks), want).max() > 0.05
    for dtype in ("float32", "bfloat16"):
        with engine(tmp_path, dtype) as eng:
            check(replay(eng, 1, toks, [70]), want, dtype)
            check(replay(eng, 2, toks, [33, 2, 30]), want, dtype)


def test_prefill_sized_steps_take_the_grouped_expert_products(tmp_path):
    """Steps of hundreds of rows sort their rows by expert into 128-row tiles (tensor-core products with the squared ReLU in the epilogue);
    the same prompt in small portions takes the per-token expert kernels: both agree with the oracle, two requests sharing a step included."""
    cfg = Z.make_config([Z.diff_layer(heads=2, kv_heads=1, dim=16, vdim=32, window=48, keep_first=2, mlp=Z.moe(experts=4, top=2, ff=40)),
                         Z.sink_layer(heads=2, kv_heads=2, dim=32, vdim=16, window=100, mlp=Z.moe(experts=9, top=3, ff=96))], width=64, vocab=70)
    W = checkpoint(tmp_path, cfg, seed=17)
    A, B = tokens_of(cfg, 420, 14), tokens_of(cfg, 270, 15)
    want_a, want_b = Z.forward(cfg, W, A), Z.forward(cfg, W, B)
    with engine(tmp_path, "bfloat16", pages=12) as eng:
        whole_a = replay(eng, 1, A, [420])
        cut_a = replay(eng, 3, A, [5, 5, 5, 5, 100, 300])
        parts = [eng.trace_step([(4, A[:40], list(range(40)))], []),
                 eng.trace_step([(4, A[40:340], list(range(300))), (5, B[:250], list(range(250)))], []),
                 eng.trace_step([(4, A[340:], list(range(80))), (5, B[250:], list(range(20)))], [4, 5])]
        mixed_a = np.concatenate([parts[0], parts[1][:300], parts[2][:80]])
        mixed_b = np.concatenate([parts[1][300:], parts[2][80:]])
    for got, want in ((whole_a, want_a), (cut_a, want_a), (mixed_a, want_a), (mixed_b, want_b)):
        check(got, want, "bfloat16")


def test_greedy_generation_through_the_scheduler(tmp_path):
    """oa_tokens_submit -> continuous batching -> greedy sampling: three requests on two sequence slots (one waits), each compared with the
    oracle's greedy continuation wherever the oracle's top-1 margin is not a near tie."""
    cfg = stack_cfg()
    W = checkpoint(tmp_path, cfg, seed=12)
    prompts = [tokens_of(cfg, n, 30 + n) for n in (9, 70, 33)]
    n_new = 12
    with engine(tmp_path, pages=6, slots=2) as eng:
        tickets = [eng.tokens_submit(p, n_new, flags=1) for p in prompts]
        outs = [eng.wait(t).token_ids for t in tickets]
        assert eng.stats()["pages_free"] == 6
    for p, out in zip(prompts, outs):
        seq = list(p)
        assert len(out) == n_new
        for tok in out:
            lg = Z.forward(cfg, W, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if int(np.argmax(lg)) != tok:
                assert top2[1] - top2[0] < 1e-3, "greedy token differs from the oracle's outside a near tie"
                break
            seq.append(tok)
