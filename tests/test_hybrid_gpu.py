"""The Ratasun hybrid family on the GPU against the slow float64 oracle (tests/hybrid_oracle.py): every mixer alone, the router, looped blocks,
and — through Engine.trace_step, the replay entry point that drives the scheduler's own batch builder, pages and state slots — prompts cut
into portions, token-by-token decoding, mixed batches and reused pages / slots.  Small random checkpoints are written per test."""
import numpy as np
import pytest

import hybrid_oracle as O

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4          # fp32 engine against the float64 oracle (relative to the logits' spread)
BF16_TOL = 0.15         # bf16 matrices / activations.  With random weights a rounding can flip an expert choice, and the recurrent layers carry
                        # that row's difference on to later rows: the bf16 runs are held to the oracle in the median and in 70 % of the rows,
                        # and exactly (SAME_TOL) to the same engine under another schedule; the fp32 runs carry the sharp comparison
SAME_TOL = 1e-2         # one engine, two schedules: a row's arithmetic does not depend on how its prompt was cut or on its batch


def engine(folder, dtype="float32", pages=8, slots=4, **kw):
    from opsagent_b200 import Engine
    return Engine(dict({"model_dir": str(folder), "dtype": dtype, "num_pages": pages, "max_seq_len": 64 * pages, "max_step_tokens": 64 * pages,
                        "max_batch": slots, "prefix_cache": 0}, **kw))


def checkpoint(tmp_path, cfg, seed=0, **kw):
    W = O.random_weights(cfg, seed, **kw)
    O.write_checkpoint(str(tmp_path), cfg, W)
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
    e = O.rel_err(got.astype(np.float64), want)
    if dtype == "float32":
        assert e.max() < F32_TOL, f"worst row {e.argmax()} differs by {e.max():.3e}"
    else:
        assert np.quantile(e, 0.7) < BF16_TOL and np.median(e) < BF16_TOL / 4, f"bf16 rows differ: median {np.median(e):.3e}, 70% {np.quantile(e, 0.7):.3e}"


MOE = O.moe()
SINGLE = {
    "attention": [O.attention_layer()],
    "attention_partial_rotation_base": [O.attention_layer(heads=3, dim=12, rot_dim=4, vdim=10, kv_rank=20, base=50.0)],
    "delta": [O.delta_layer()],
    "delta_equal_heads": [O.delta_layer(heads=2, kv_heads=2, dim=8, vdim=8, conv=2)],
    "mamba": [O.mamba_layer()],
    "mamba_one_group_three_norm_groups": [O.mamba_layer(heads=3, vdim=8, state=12, groups=1, norm_groups=3, conv=5)],
    "attention_moe": [O.attention_layer(mlp=MOE)],
    "moe_top1_all_groups": [O.mamba_layer(mlp=O.moe(experts=4, top=1, groups=2, keep=2, ff=16, scale=1.0))],
    "moe_single_member_groups": [O.delta_layer(mlp=O.moe(experts=5, top=2, groups=5, keep=3, ff=20, scale=2.5))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = O.make_config(SINGLE[name], width=40, vocab=77, logit_scale=1.5)
    W = checkpoint(tmp_path, cfg, seed=len(name))
    toks = tokens_of(cfg, 70, 1)                       # crosses a page border
    want = O.forward(cfg, W, toks)
    with engine(tmp_path, dtype) as eng:
        check(replay(eng, 1, toks, [70]), want, dtype)           # whole prompt
        check(replay(eng, 2, toks, [1, 1, 2, 3, 57, 2]), want, dtype)   # the first tokens alone, short portions, then token by token


def hybrid_cfg(loop=True):
    layers = [O.attention_layer(mlp=MOE), O.delta_layer(mlp=MOE), O.mamba_layer(mlp=None), O.attention_layer(heads=1, dim=8, rot_dim=8, vdim=32, kv_rank=16, mlp=MOE)]
    return O.make_config(layers, loop={"start": 1, "stop": 3, "times": 2} if loop else None, logit_scale=2.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_decoding_match_the_whole_prompt(tmp_path, dtype):
    cfg = hybrid_cfg()
    W = checkpoint(tmp_path, cfg, seed=3)
    toks = tokens_of(cfg, 140, 2)
    want = O.forward(cfg, W, toks)
    with engine(tmp_path, dtype) as eng:
        for cuts in ([140], [2, 62, 1, 2, 61, 12], [63, 2, 64], [5], [127, 1, 1, 11], [64, 64, 2, 2, 2, 2, 2, 2]):
            check(replay(eng, 7, toks, cuts), want, dtype)


def test_looped_attention_has_a_cache_per_pass_and_no_loop_runs(tmp_path):
    layers = [O.delta_layer(mlp=MOE), O.attention_layer(mlp=None), O.mamba_layer(mlp=MOE)]
    for k, loop in enumerate([{"start": 0, "stop": 3, "times": 3}, {"start": 1, "stop": 2, "times": 1}, None]):
        cfg = O.make_config(layers, width=56, vocab=90, loop=loop)
        folder = tmp_path / str(k)
        W = checkpoint(folder, cfg, seed=10 + k)
        toks = tokens_of(cfg, 75, 4)
        with engine(folder) as eng:
            check(replay(eng, 1, toks, [3, 61, 2]), O.forward(cfg, W, toks), "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(tmp_path, dtype):
    """Three requests at different stages share every step (a prompt portion beside single tokens); then later requests take over the pages
    and the two state slots of finished ones: a stale state or cache row would show."""
    cfg = hybrid_cfg()
    W = checkpoint(tmp_path, cfg, seed=5)
    lens = {1: 100, 2: 37, 3: 66, 4: 90, 5: 20}
    toks = {r: tokens_of(cfg, n, 20 + r) for r, n in lens.items()}
    want = {r: O.forward(cfg, W, toks[r]) for r in lens}
    got = {r: [] for r in lens}
    at = {r: 0 for r in lens}
    with engine(tmp_path, dtype, pages=4, slots=2) as eng:
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
        step([(1, 3), (2, 7)])                        # 2 ends: its page and slot are free
        step([(1, 36), (5, 2)])                       # 1 ends, 5 starts in 2's slot
        step([(5, 18), (3, 64)])                      # 5 ends; 3 takes 1's slot, filling exactly one page
        step([(3, 2), (4, 2)])                        # 3 ends on a page's second token; 4 starts
        while at[4] < lens[4]:
            step([(4, 29)])
        assert eng.stats()["pages_free"] == 4
        for r in lens:                                # each alone, whole, in the same engine: the same rows up to rounding
            alone = replay(eng, 10 + r, toks[r], [lens[r]])
            assert O.rel_err(np.concatenate(got[r]).astype(np.float64), alone.astype(np.float64)).max() < SAME_TOL
    for r in lens:
        check(np.concatenate(got[r]), want[r], dtype)


def test_a_far_key_decides_and_is_found_through_pages_and_decoding(tmp_path):
    """Sharp attention: single keys dominate, also hundreds of tokens back.  The oracle itself shows the sensitivity (without the first page
    the answer changes by far more than the tolerance), and the engine must agree with it in prompts and in decoding."""
    cfg = O.make_config([O.attention_layer(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, base=500000.0), O.attention_layer(mlp=MOE)], width=48, vocab=64)
    W = checkpoint(tmp_path, cfg, seed=8, sharp=7.0)
    toks = tokens_of(cfg, 330, 6)
    want = O.forward(cfg, W, toks)
    without_first_page = O.forward(cfg, W, toks[64:])
    assert O.rel_err(without_first_page[-40:], want[-40:]).max() > 50 * F32_TOL
    with engine(tmp_path, pages=6) as eng:
        check(replay(eng, 1, toks, [330]), want, "float32")
        check(replay(eng, 2, toks, [255, 2, 63]), want, "float32")      # decodes across the borders at 256 and 320


def test_long_decoding(tmp_path):
    cfg = hybrid_cfg()
    W = checkpoint(tmp_path, cfg, seed=9)
    toks = tokens_of(cfg, 200, 7)
    with engine(tmp_path) as eng:
        check(replay(eng, 1, toks, [3]), O.forward(cfg, W, toks), "float32")     # 197 single-token steps over three page borders


def test_bf16_tensor_core_path_and_plain_path_agree_with_the_oracle(tmp_path):
    cfg = hybrid_cfg()
    W = checkpoint(tmp_path, cfg, seed=11)
    toks = tokens_of(cfg, 150, 8)
    want = O.forward(cfg, W, toks)
    for tc in (0, 1):
        with engine(tmp_path, "bfloat16", hy_tensor_core=tc) as eng:
            check(replay(eng, 1, toks, [150]), want, "bfloat16")
            check(replay(eng, 2, toks, [130]), want, "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_fit_no_tile(tmp_path, dtype):
    """Widths, ranks and head sizes that are multiples of nothing: every product falls back to the plain GEMM, attention to the one-query
    kernel, the recurrences to the shared-memory kernel; one-tap and five-tap convolutions; one expert group; a single chosen expert."""
    layers = [O.attention_layer(heads=3, dim=6, rot_dim=4, vdim=10, kv_rank=20, mlp=O.moe(experts=3, top=1, groups=1, keep=1, ff=10, scale=0.7)),
              O.delta_layer(heads=3, kv_heads=3, dim=6, vdim=10, conv=1, mlp=None),
              O.mamba_layer(heads=2, vdim=6, state=6, groups=2, norm_groups=2, conv=5, mlp=O.moe(experts=6, top=3, groups=2, keep=2, ff=21, scale=1.0)),
              O.delta_layer(heads=4, kv_heads=2, dim=132, vdim=12, conv=3, mlp=None)]          # dim beyond the register kernel
    cfg = O.make_config(layers, width=36, vocab=51, loop={"start": 1, "stop": 3, "times": 2}, logit_scale=0.5)
    W = checkpoint(tmp_path, cfg, seed=21, low_rank=5)
    toks = tokens_of(cfg, 90, 11)
    want = O.forward(cfg, W, toks)
    with engine(tmp_path, dtype) as eng:
        check(replay(eng, 1, toks, [90]), want, dtype)
        check(replay(eng, 2, toks, [2, 62, 3, 20]), want, dtype)


def test_tensor_core_attention_sizes(tmp_path):
    """Latent sizes that take the mma.sync attention kernel (rank a multiple of 64, rank + rotated a multiple of 16) and, for prompts of 256
    rows and more, the per-head tensor-core absorption / up-projection products: whole prompts, portions that straddle the 64-query tiles and
    the 16- or 32-row cache tiles, and decoding (also with the cache rows of a row cut into parts), against the oracle and against the plain kernels (hy_tensor_core = 0)."""
    layers = [O.attention_layer(heads=4, dim=16, rot_dim=16, vdim=16, kv_rank=64), O.attention_layer(heads=3, dim=24, rot_dim=32, vdim=8, kv_rank=128, base=500.0)]
    cfg = O.make_config(layers, width=64, vocab=96)
    W = checkpoint(tmp_path, cfg, seed=13, sharp=3.0)
    toks = tokens_of(cfg, 600, 9)
    want = O.forward(cfg, W, toks)
    outs = {}
    for tc in (1, 0):
        with engine(tmp_path, "bfloat16", pages=10, hy_tensor_core=tc) as eng:     # the last tokens decode one by one at contexts past 512: their cache rows are cut into parts
            outs[tc] = [replay(eng, 1, toks, [600]), replay(eng, 2, toks, [17, 33, 63, 130, 41, 290]), replay(eng, 3, toks, [500])]
    for tc in (1, 0):
        for got in outs[tc]:
            e = O.rel_err(got.astype(np.float64), want)
            assert np.quantile(e, 0.95) < 0.06 and e.max() < 0.2, f"tensor cores {tc}: 95% {np.quantile(e, 0.95):.3e}, worst {e.max():.3e}"
    for got in outs[1][1:]:                           # schedules agree more closely than bf16 agrees with the oracle (a cut row sums its parts
        assert O.rel_err(got.astype(np.float64), outs[1][0].astype(np.float64)).max() < 3 * SAME_TOL      # in another order, and these scores are sharp)


def test_wide_latent_takes_the_small_cache_tile(tmp_path):
    """A latent row so wide that only the 16-row cache tile of the tensor-core kernel fits shared memory (the 32-row tile does not): decoding
    rows and short portions behind a long context (absorbed form) and whole prompts (prefill form) against the oracle."""
    cfg = O.make_config([O.attention_layer(heads=2, dim=16, rot_dim=32, vdim=16, kv_rank=768)], width=64, vocab=96)
    W = checkpoint(tmp_path, cfg, seed=19)
    toks = tokens_of(cfg, 180, 12)
    want = O.forward(cfg, W, toks)
    with engine(tmp_path, "bfloat16", pages=4) as eng:
        for cuts in ([180], [150, 5, 3, 2], [40]):
            e = O.rel_err(replay(eng, 1, toks, cuts).astype(np.float64), want)
            assert np.quantile(e, 0.95) < 0.06 and e.max() < 0.2, f"cuts {cuts}: 95% {np.quantile(e, 0.95):.3e}, worst {e.max():.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_router_with_negative_choice_scores(tmp_path, dtype):
    """Corrections far below zero make every choice score negative, so an expert of a dropped group must count as minus infinity (a zero
    would beat every kept expert); corrections that differ by more than the scores' range make the correction, not the score, pick the
    experts, while the weights still come from the uncorrected scores.  The oracle shows that both matter before the engine is asked."""
    mlp = O.moe(experts=8, top=3, groups=4, keep=2, ff=16, scale=1.7)
    cfg = O.make_config([O.mamba_layer(mlp=mlp), O.attention_layer(mlp=mlp)], width=40, vocab=60)
    W = O.random_weights(cfg, 23)
    rng = np.random.default_rng(5)
    for i in range(2):
        W["l%d.mlp.correction" % i] = O.bf16_round(-3.0 + 1.5 * rng.standard_normal(8)).astype(np.float64)
    O.write_checkpoint(str(tmp_path), cfg, W)
    toks = tokens_of(cfg, 70, 3)
    want = O.forward(cfg, W, toks)
    plain = dict(W)
    for i in range(2):
        plain["l%d.mlp.correction" % i] = np.zeros(8)
    assert O.rel_err(O.forward(cfg, plain, toks), want).max() > 0.05          # the corrections change the answer
    with engine(tmp_path, dtype) as eng:
        check(replay(eng, 1, toks, [70]), want, dtype)
        check(replay(eng, 2, toks, [33, 2, 30]), want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_recurrence_with_rows_split_over_warps(tmp_path, dtype):
    """State sizes beyond 32 rows split a column's rows over a CTA's four warps: key sizes that fill the 64- and 128-row variants and one
    that leaves padding rows, value sizes that are no multiple of the 32 columns of a CTA; whole, in portions, and token by token (a
    one-token step joins its read-out after the loop), two sequences in one step."""
    layers = [O.delta_layer(heads=2, kv_heads=1, dim=64, vdim=40, conv=3), O.mamba_layer(heads=2, vdim=24, state=128, groups=1, norm_groups=1, conv=2),
              O.delta_layer(heads=3, kv_heads=3, dim=100, vdim=8, conv=2), O.mamba_layer(heads=4, vdim=36, state=48, groups=2, norm_groups=2, conv=4)]
    cfg = O.make_config(layers, width=64, vocab=70)
    W = checkpoint(tmp_path, cfg, seed=29)
    A, B = tokens_of(cfg, 100, 16), tokens_of(cfg, 45, 17)
    want_a, want_b = O.forward(cfg, W, A), O.forward(cfg, W, B)
    with engine(tmp_path, dtype, pages=6, slots=2) as eng:
        check(replay(eng, 1, A, [100]), want_a, dtype)
        check(replay(eng, 2, A, [1, 2, 61, 3, 20]), want_a, dtype)
        parts = [eng.trace_step([(3, A[:70], list(range(70))), (4, B[:5], list(range(5)))], []),
                 eng.trace_step([(3, A[70:71], [0]), (4, B[5:], list(range(40)))], [4]),
                 eng.trace_step([(3, A[71:], list(range(29)))], [3])]
        check(np.concatenate([parts[0][:70], parts[1][:1], parts[2]]), want_a, dtype)
        check(np.concatenate([parts[0][70:], parts[1][1:]]), want_b, dtype)


def test_prefill_sized_steps_of_the_recurrent_layers(tmp_path):
    """Steps of 512 rows and more take the convolution kernel that walks 16 rows per thread, smaller steps the one-row kernel: a prompt
    whole, the same prompt in portions below that size, and two requests sharing a large step (one continuing from its carried tail, the
    other starting in the middle of a 16-row block) agree with each other and with the oracle.  No routed experts: nothing can flip."""
    layers = [O.delta_layer(heads=4, kv_heads=2, dim=16, vdim=32, conv=4), O.mamba_layer(heads=4, vdim=16, state=16, groups=2, norm_groups=2, conv=3),
              O.delta_layer(heads=2, kv_heads=2, dim=32, vdim=64, conv=2), O.mamba_layer(heads=2, vdim=64, state=24, groups=1, norm_groups=1, conv=4)]
    cfg = O.make_config(layers, width=64, vocab=70)
    W = checkpoint(tmp_path, cfg, seed=17)
    A, B = tokens_of(cfg, 620, 14), tokens_of(cfg, 270, 15)
    want_a, want_b = O.forward(cfg, W, A), O.forward(cfg, W, B)
    with engine(tmp_path, "bfloat16", pages=16, slots=2) as eng:
        whole_a, whole_b = replay(eng, 1, A, [620]), replay(eng, 2, B, [270])
        cut_a = replay(eng, 3, A, [100, 100, 100, 100, 100, 100, 18])
        parts = [eng.trace_step([(4, A[:40], list(range(40)))], []),
                 eng.trace_step([(4, A[40:340], list(range(300))), (5, B[:250], list(range(250)))], []),
                 eng.trace_step([(4, A[340:], list(range(280))), (5, B[250:], list(range(20)))], [4, 5])]
        mixed_a = np.concatenate([parts[0], parts[1][:300], parts[2][:280]])
        mixed_b = np.concatenate([parts[1][300:], parts[2][280:]])
    for got, ref in ((cut_a, whole_a), (mixed_a, whole_a), (mixed_b, whole_b)):
        assert O.rel_err(got.astype(np.float64), ref.astype(np.float64)).max() < SAME_TOL
    for got, want in ((whole_a, want_a), (whole_b, want_b), (mixed_a, want_a), (mixed_b, want_b)):
        assert O.rel_err(got.astype(np.float64), want).max() < BF16_TOL


def test_greedy_generation_through_the_scheduler(tmp_path):
    """oa_tokens_submit -> continuous batching -> greedy sampling: three requests on two state slots (one waits for a slot), each compared
    with the oracle's greedy continuation wherever the oracle's top-1 margin is not a near tie."""
    cfg = hybrid_cfg()
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
            lg = O.forward(cfg, W, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if int(np.argmax(lg)) != tok:
                assert top2[1] - top2[0] < 1e-3, "greedy token differs from the oracle's outside a near tie"
                break
            seq.append(tok)
