"""Sumozen on the device against the plain implementation (``plain_sumozen``, float64).

Every test makes its own small configuration and random weights.  32-bit runs must agree within
1e-4 at every token; bfloat16 runs within 4 % of the logits' spread in the root mean square.  The schedules cut the same
requests in different ways: a request's logits must not depend on the cut, on the rest of the
batch, or on which pages and slots it got."""

import numpy as np
import pytest
import torch

import plain_sumozen as plain
import sumozen_helpers as sz
from engine_helpers import (F32_ATOL, bf16_atol, random_tokens, run_schedule, schedule_mixed, schedule_portions,
                            schedule_tail_one_by_one, schedule_whole)

pytestmark = pytest.mark.gpu


def engine_for(folder, dtype="float32", **options):
    from mini_llm_b200.engine import Engine
    options.setdefault("page_size", 8)
    options.setdefault("max_requests", 4)
    options.setdefault("cache_tokens", 1024)
    return Engine(folder, dtype=dtype, **options)


def check(engine, folder, requests, steps, atol=F32_ATOL):
    got = run_schedule(engine, requests, steps)
    for name, tokens in requests.items():
        expected = sz.plain_logits(folder, tokens)
        worst = np.abs(got[name] - expected).max(axis=1)
        assert worst.max() <= atol, f"request {name}: first wrong token {int(np.argmax(worst > atol))} of {len(tokens)}, off by {worst.max():.2e}"
    engine.cache.check()


def dev(values, dtype=torch.float32):
    return torch.tensor(np.asarray(values), dtype=dtype, device="cuda")


# ---- each mechanism alone ----------------------------------------------------------------------

@pytest.mark.parametrize("layer", [
    sz.parallel(right_scale=0.0, mlp=None),
    sz.parallel(right_scale=0.0, mlp=None, heads=6, kv_heads=1, dim=8, vdim=40, taps=1, rot_dims=0, scaling=None, softcap=None),
    sz.parallel(right_scale=0.0, mlp=None, heads=2, kv_heads=2, dim=24, vdim=8, taps=5, rot_dims=24, softcap=0.8, scale=2.0),
    sz.parallel(left_scale=0.0, mlp=None),
    sz.parallel(left_scale=0.0, mlp=None, r_heads=1, r_kv_heads=1, r_dim=40, r_vdim=33, r_taps=1),
    sz.parallel(left_scale=0.0, mlp=None, r_heads=6, r_kv_heads=2, r_dim=4, r_vdim=70, r_taps=2),
    sz.parallel(),
    sz.mamba(mlp=None), sz.mamba(mlp=None, heads=1, vdim=33, state=5, groups=1, norm_groups=1, taps=1),
    sz.mamba(mlp=None, heads=6, vdim=8, state=40, groups=6, norm_groups=6, taps=2),
    sz.mamba(mlp=sz.moe(experts=7, top=1, ff=12, shared=None)), sz.mamba(mlp=sz.moe(experts=3, top=3, ff=40, shared=8)),
], ids=["attention", "attention_one_kv_head_no_rotation_no_cap_one_tap", "attention_hard_cap_all_rotated", "delta",
        "delta_one_head_one_tap", "delta_three_heads_a_key", "both_sides", "state_space", "state_space_one_head",
        "state_space_group_per_head", "experts_top_one_no_shared", "experts_all_chosen"])
def test_one_layer_of_each_kind(tmp_path, layer):
    folder = sz.make_model(str(tmp_path / "m"), sz.config([layer]), seed=3, matrix_scale=3.0)
    engine = engine_for(folder)
    requests = {"a": random_tokens(1, 37, 211), "b": random_tokens(2, 1, 211), "c": random_tokens(3, 2, 211)}
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_portions(requests))


def test_residual_stream_after_every_layer(tmp_path):
    from mini_llm_b200.engine import StepEntry
    folder = sz.make_model(str(tmp_path / "m"), sz.full_stack(), seed=5, matrix_scale=2.0)
    engine = engine_for(folder)
    tokens = random_tokens(4, 29, 211)
    streams = []
    sz.plain_logits(folder, tokens, streams)
    slot = engine.open_request()
    engine.step([StepEntry(slot, tokens, [28])], dump_hidden=True)
    assert len(engine.hidden_dump) == len(streams) + 1
    for index, expected in enumerate(streams):
        np.testing.assert_allclose(engine.hidden_dump[index + 1].cpu().numpy(), expected, rtol=0,
                                   atol=1e-4 * np.abs(expected).max(), err_msg=f"after layer {index}")
    engine.close_request(slot)


# ---- the same tokens, cut differently -----------------------------------------------------------

def test_prompt_against_token_by_token_and_portions(tmp_path):
    folder = sz.make_model(str(tmp_path / "m"), sz.full_stack(), seed=7, bend=sz.sharpen(6.0), matrix_scale=2.0)
    engine = engine_for(folder)
    requests = {"a": random_tokens(11, 45, 211), "b": random_tokens(12, 7, 211)}
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=45))        # every token alone, from the first
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=5))
    check(engine, folder, requests, schedule_portions(requests))
    check(engine, folder, requests, schedule_portions(requests, sizes=(2, 2, 3, 2, 17)))
    assert engine.step_kinds["replayed"] > 0          # steps of one shape were replayed from a captured graph


def test_mixed_batches_and_reuse_of_pages_and_slots(tmp_path):
    """Six requests through three slots and a page pool that holds less than their sum: pages
    and slots are given back and used again (and poisoned in between), portions run beside
    single tokens; every request must come out as it does alone."""
    folder = sz.make_model(str(tmp_path / "m"), sz.full_stack(), seed=9, bend=sz.sharpen(6.0), matrix_scale=2.0)
    lengths = {"a": 61, "b": 9, "c": 33, "d": 2, "e": 40, "f": 18}
    requests = {name: random_tokens(20 + i, n, 211) for i, (name, n) in enumerate(lengths.items())}
    prompts = {"a": 40, "b": 9, "c": 20, "d": 1, "e": 40, "f": 3}
    engine = engine_for(folder, max_requests=3, cache_tokens=160, debug_poison=True)
    check(engine, folder, requests, schedule_mixed(requests, prompts, max_live=3))
    check(engine, folder, requests, schedule_mixed(requests, prompts, max_live=2, portion_sizes=(2, 11, 3)))
    assert not any(engine.cache.pages_in_use()) and engine.cache.free_slots == 3


def test_a_far_key_decides(tmp_path):
    """One early token's key is made to match the last token's query, and its value to stand out:
    the logits then hang on that single far key among hundreds (behind many page borders), in a
    prompt, in portions and when the last tokens are decoded alone.  The same key one place off
    (a wrong rotation or a key stored in a neighbour's place) would not match."""
    layer = sz.parallel(heads=2, kv_heads=1, dim=8, vdim=8, taps=1, rot_dims=4, base=50.0, scaling=None, scale=1.0, softcap=30.0,
                        right_scale=0.0, mlp=None)
    raw = sz.config([layer], vocab=64, width=32)

    def bend(t):
        # only tokens 5 and 9 have anything in the first eight channels; key entry 7 (not rotated) of
        # the one key head reads them, and so does query entry 7 of head 0, with the other sign for
        # token 9: token 9's query finds token 5's key.  The taps are the identity.
        t["embed"][:, :8] = 0.0
        t["embed"][5, :8] = 2.0
        t["embed"][9, :8] = -2.0
        t["l0.norm1"][:] = 0.0
        for name in ("q", "k", "v"):
            t[f"l0.mix.left.{name}.conv"][:] = 1.0
            t[f"l0.mix.left.{name}.b"][:] = 0.0
        t["l0.mix.left.k"][7] = 0.0
        t["l0.mix.left.k"][7, :8] = 2.0
        t["l0.mix.left.q"][7] = 0.0
        t["l0.mix.left.q"][7, :8] = -2.0
    folder = sz.make_model(str(tmp_path / "m"), raw, seed=13, bend=bend, matrix_scale=2.0)
    rng = np.random.default_rng(0)
    base = [int(t) for t in rng.integers(10, 64, 300)]
    base[-1] = 9
    with_key, without = list(base), list(base)
    with_key[3] = 5
    assert np.abs(sz.plain_logits(folder, with_key)[-1] - sz.plain_logits(folder, without)[-1]).max() > 0.1
    engine = engine_for(folder)
    for tokens in (with_key, without):
        requests = {"r": tokens}
        check(engine, folder, requests, schedule_whole(requests))
        check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=3))
        check(engine, folder, requests, schedule_portions(requests, sizes=(8, 7, 9, 64, 2)))


def test_an_old_write_is_read_back_and_replaced(tmp_path):
    """The delta rule with decays bent to almost 1 in one head and to a fast fall in the other, and
    write gates near 1: what an early token wrote is still read two hundred tokens later, and a later
    token with the same key replaces it.  Long decoding, token by token, against the whole prompt."""
    layer = sz.parallel(left_scale=0.0, r_heads=2, r_kv_heads=1, r_dim=8, r_vdim=8, r_taps=2, mlp=None)
    raw = sz.config([layer, sz.mamba(heads=2, vdim=8, state=8, groups=1, norm_groups=2, taps=2, mlp=None)], width=32, vocab=97)

    def bend(t):
        t["l0.mix.right.A_log"][:] = [-9.0, 1.5]
        t["l0.mix.right.dt_bias"][:] = [-2.0, 1.0]
        t["l0.mix.right.b"] *= 30.0                      # write gates at both ends
        t["l1.mix.A_log"][:] = [-8.0, 0.5]
        t["l1.mix.dt_bias"][:] = [0.5, 2.0]
        t["l1.mix.D"][:] = [1.5, -0.5]
    folder = sz.make_model(str(tmp_path / "m"), raw, seed=17, bend=bend, matrix_scale=2.0)
    engine = engine_for(folder)
    requests = {"long": random_tokens(31, 221, 97)}
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=220))
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_portions(requests, sizes=(16, 17, 15, 2, 33)))


def all_experts(raw):
    """The same stack with every expert chosen for every token: the scores still weigh the experts'
    inputs, but no choice hangs on a near tie, which rounding to bfloat16 may turn (the 32-bit tests
    cover the choice itself)."""
    for layer in raw["layers"]:
        if layer["mlp"] is not None:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return raw


def check_rounding(engine, folder, requests, steps, share=0.04):
    """bfloat16 against the plain model: over a request, the root mean square of the difference stays
    below ``share`` of the logits' standard deviation.  (Not a bound on every token: where a
    recurrence's read nearly cancels its write, the rounding of its inputs shows many times over in
    that token and is carried on to the later tokens of the request; the 32-bit runs bound every token.)"""
    got = run_schedule(engine, requests, steps)
    for name, tokens in requests.items():
        expected = sz.plain_logits(folder, tokens)
        ratio = float(np.sqrt(((got[name] - expected) ** 2).mean()) / expected.std())
        assert ratio <= share, f"request {name}: root mean square of the difference is {ratio:.3f} of the logits' spread"
    engine.cache.check()


def test_bfloat16_follows_within_its_rounding(tmp_path):
    folder = sz.make_model(str(tmp_path / "m"), all_experts(sz.full_stack(width=128)), seed=19, bfloat16_values=True)
    engine = engine_for(folder, dtype="bfloat16")
    requests = {"a": random_tokens(41, 140, 211), "b": random_tokens(42, 12, 211), "c": random_tokens(43, 70, 211)}
    check_rounding(engine, folder, requests, schedule_whole(requests))
    check_rounding(engine, folder, requests, schedule_mixed(requests, {"a": 100, "b": 6, "c": 64}, max_live=3))
    check_rounding(engine, folder, requests, schedule_tail_one_by_one(requests, tail=10))
    chosen = {kernel for key, kernel in engine.kernels.choices.items() if key[0] in ("capped_attention", "linear")}
    assert {"capped_attention_tiled", "capped_attention_plain", "gemm_tcgen05"} <= chosen


def test_bfloat16_with_sizes_no_fast_kernel_takes(tmp_path):
    """A width that is no multiple of 8, key sizes of 6 and 10, a state of 5: every product and the
    attention fall back to kernels that take any size, in bfloat16 too."""
    raw = sz.config([sz.parallel(heads=3, kv_heads=1, dim=10, vdim=14, rot_dims=6, r_heads=2, r_kv_heads=2, r_dim=6, r_vdim=10),
                     sz.mamba(heads=3, vdim=7, state=5, groups=3, norm_groups=1, taps=5, mlp=sz.moe(experts=3, top=2, ff=9, shared=5))],
                    width=100, vocab=203)
    folder = sz.make_model(str(tmp_path / "m"), all_experts(raw), seed=29, bfloat16_values=True)
    requests = {"a": random_tokens(61, 150, 203), "b": random_tokens(62, 3, 203), "c": random_tokens(63, 40, 203)}
    engine = engine_for(folder, dtype="bfloat16")
    check_rounding(engine, folder, requests, schedule_whole(requests))
    check_rounding(engine, folder, requests, schedule_mixed(requests, {"a": 130, "b": 2, "c": 33}, max_live=3))
    chosen = {kernel for key, kernel in engine.kernels.choices.items() if key[0] in ("capped_attention", "linear")}
    assert chosen == {"capped_attention_plain", "linear_plain"}
    check(engine_for(folder), folder, requests, schedule_portions(requests))


def test_greedy_generation_through_the_scheduler(tmp_path):
    from mini_llm_b200.generate import generate
    folder = sz.make_model(str(tmp_path / "m"), sz.full_stack(), seed=23, matrix_scale=3.0)
    model_config, tensors = plain.load_model(folder)
    prompts = [random_tokens(50 + i, n, 211) for i, n in enumerate((3, 19, 1, 30, 8))]
    got = generate(folder, prompts, max_new_tokens=12, temperature=0.0, dtype="float32", page_size=8, max_sessions=3,
                   cache_tokens=256, max_prefill_chunk=7)
    for prompt, generated in zip(prompts, got):
        tokens = list(prompt)
        for index, token in enumerate(generated):
            logits = plain.forward(model_config, tensors, tokens)[-1]
            ordered = np.sort(logits)
            if ordered[-1] - ordered[-2] < 1e-3:
                break                                   # a near tie: either token is right, and the paths part here
            assert token == int(np.argmax(logits)), f"generated token {index}"
            tokens.append(token)


# ---- the mechanisms' kernels by themselves ------------------------------------------------------

def test_norm_kernel_with_its_gates():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(1)
    x, gate, gain = rng.normal(0, 2, (9, 120)), rng.normal(0, 2, (9, 120)), rng.uniform(0.5, 1.5, 120)

    def norm(values, groups, eps):
        parts = values.reshape(9, groups, -1)
        return (parts / np.sqrt((parts * parts).mean(-1, keepdims=True) + eps)).reshape(9, 120) * gain
    for groups in (1, 3, 8):
        out = torch.empty((9, 120), dtype=torch.float32, device="cuda")
        ops.grouped_rms_norm(out, dev(x), dev(gain), groups, 1e-3, gate=dev(gate), gate_mode="silu")
        np.testing.assert_allclose(out.cpu().numpy(), norm(x, groups, 1e-3) * plain.silu(gate), atol=3e-6)
        ops.grouped_rms_norm(out, dev(x), dev(gain), groups, 1e-3, gate=dev(gate), gate_mode="silu_before")
        np.testing.assert_allclose(out.cpu().numpy(), norm(x * plain.silu(gate), groups, 1e-3), atol=3e-6)


def _cut_batches(lengths, cuts):
    """Steps over requests 0 and 1 (in slots 2 and 0): per step the rows and the entry arrays."""
    done = {r: 0 for r in lengths}
    for cut in cuts:
        step = dict(positions=[], token_item=[], slots=[], starts=[], offsets=[], counts=[], rows=[])
        for item, (request, n) in enumerate(cut.items()):
            step["offsets"].append(len(step["positions"]))
            step["rows"].append((request, done[request], n))
            step["positions"] += list(range(done[request], done[request] + n))
            step["token_item"] += [item] * n
            step["slots"].append(2 if request == 0 else 0)
            step["starts"].append(done[request])
            step["counts"].append(n)
            done[request] += n
        yield step


def test_taps_kernel_with_bias_and_activation_over_cuts():
    """The convolution alone (no identity), with a bias and silu, on a column range of a wider
    buffer, two requests in one batch, portions of one, two and more tokens."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(2)
    width, taps, extra = 20, 4, 7
    h = {0: rng.normal(0, 1, (11, width)), 1: rng.normal(0, 1, (5, width))}
    w, bias = rng.normal(0, 0.5, (width, taps)), rng.normal(0, 0.5, width)
    expected = {i: plain.silu(plain.causal_taps(h[i], w, bias)) for i in h}
    state = torch.zeros((3, taps - 1, width), dtype=torch.float32, device="cuda")
    got = {0: [], 1: []}
    for step in _cut_batches(h, ({0: 1, 1: 2}, {0: 2, 1: 1}, {0: 5}, {1: 2, 0: 3})):
        rows = np.concatenate([h[r][first:first + n] for r, first, n in step["rows"]])
        wide = dev(np.concatenate([rng.normal(0, 1, (rows.shape[0], extra)), rows], axis=1))
        out = torch.full((rows.shape[0], width + 3), float("nan"), device="cuda")
        ints = lambda key: dev(step[key], torch.int32)
        ops.causal_taps(out[:, :width], wide[:, extra:], dev(w), state, ints("positions"), ints("token_item"), ints("slots"),
                        ints("starts"), ints("offsets"), ints("counts"), identity=False, bias=dev(bias), silu=True)
        for item, (r, first, n) in enumerate(step["rows"]):
            got[r].append(out[step["offsets"][item]:step["offsets"][item] + n, :width].cpu().numpy())
    for request in (0, 1):
        np.testing.assert_allclose(np.concatenate(got[request]), expected[request], atol=3e-6)


@pytest.mark.parametrize("heads, qk_heads, dim, vdim", [(2, 1, 12, 37), (3, 3, 40, 8), (4, 2, 70, 33), (1, 1, 130, 20),
                                                        (2, 2, 300, 6), (60, 2, 40, 70), (80, 2, 40, 70), (60, 3, 100, 40),
                                                        (80, 4, 100, 40)])
def test_recurrence_kernel_carries_its_state(heads, qk_heads, dim, vdim):
    """Both forms, a sequence cut in six (down to one token), against the token-by-token formulas.
    (With 60 and 80 heads a thread of the kernel takes four columns of the state.)"""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(dim)
    n = 100
    q, k = rng.normal(0, 1, (n, qk_heads * dim)), rng.normal(0, 1, (n, qk_heads * dim))
    v = rng.normal(0, 1, (n, heads * vdim))
    gate_a, gate_b = rng.normal(0, 2, (n, heads)), rng.normal(0, 3, (n, heads))
    log_rate, bias, skip = rng.normal(-1, 1, heads), rng.normal(0, 1, heads), rng.normal(0, 1, heads)
    for delta in (True, False):
        expected = np.zeros((n, heads, vdim))
        for head in range(heads):
            g = head // (heads // qk_heads)
            S = np.zeros((dim, vdim))
            for t in range(n):
                qt, kt = q[t, g * dim:(g + 1) * dim], k[t, g * dim:(g + 1) * dim]
                vt = v[t, head * vdim:(head + 1) * vdim]
                step = plain.softplus(gate_a[t, head] + bias[head])
                a = np.exp(-np.exp(log_rate[head]) * step)
                if delta:
                    qt = qt / np.sqrt((qt * qt).sum() + 1e-6) * 0.5
                    kt = kt / np.sqrt((kt * kt).sum() + 1e-6)
                    S = a * S
                    S = S + np.outer(kt, plain.sigmoid(gate_b[t, head]) * (vt - S.T @ kt))
                    expected[t, head] = S.T @ qt
                else:
                    S = a * S + step * np.outer(kt, vt)
                    expected[t, head] = S.T @ qt + skip[head] * vt
        state = torch.zeros((2, heads * dim * vdim), dtype=torch.float32, device="cuda")
        out = torch.empty((n, heads * vdim), dtype=torch.float32, device="cuda")
        for first, count in ((0, 1), (1, 9), (10, 3), (13, 10), (23, 32), (55, 45)):
            # entry 0 is another request with no tokens in this step; entry 1 is ours, in slot 1.  The step
            # holds the portion's rows only: short portions take the kernel's form for few tokens an entry.
            rows = slice(first, first + count)
            ops.linear_recurrence(out[rows], dev(q[rows]), dev(k[rows]), dev(v[rows]), dev(gate_a[rows]),
                                  dev(gate_b[rows]) if delta else None, dev(log_rate), dev(bias), state,
                                  dev([0, 1], torch.int32), dev([0, 0], torch.int32), dev([0, count], torch.int32), heads,
                                  qk_heads, dim, vdim, delta, unit_norm=delta, q_scale=0.5 if delta else 1.0,
                                  skip=None if delta else dev(skip))
        # (32-bit sums: an entry's rounding follows the largest values that went into it, not its own)
        np.testing.assert_allclose(out.cpu().numpy(), expected.reshape(n, heads * vdim), rtol=5e-5,
                                   atol=5e-6 * max(4.0, float(np.abs(expected).max())), err_msg=f"delta {delta}")
        assert float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, cap", [(4, 2, 16, 24, 5.0), (1, 1, 8, 8, 0.0), (6, 1, 64, 32, 2.0),
                                                              (40, 2, 12, 72, 0.0), (3, 3, 128, 256, 9.0), (128, 2, 64, 64, 3.0)])
def test_attention_in_tiles_against_one_block_per_row(heads, kv_heads, dim, vdim, cap):
    """Prompt portions of three requests in one batch (one of them three tokens, so that tiles hold
    tokens of several requests), pages scattered over the pool: the tiled kernel must give what the
    kernel with one block per (token, head) gives, and that one what the formula gives.  (With 40
    and 128 heads the step has rows enough for the tiles of four rows a warp.)"""
    from mini_llm_b200.kernels import ops
    torch.manual_seed(heads * 1000 + dim)
    page_size = 8
    lengths, new = [150, 9, 77], [150, 3, 40]                 # cached + new tokens; tokens of this step
    blocks = [-(-n // page_size) for n in lengths]
    k_pages = torch.randn(sum(blocks) + 1, page_size, kv_heads, dim, device="cuda")
    v_pages = torch.randn(sum(blocks) + 1, page_size, kv_heads, vdim, device="cuda")
    order = torch.randperm(sum(blocks)).tolist()              # pages scattered over the pool
    table = torch.zeros(3, max(blocks), dtype=torch.int32)
    at = 0
    for i, count in enumerate(blocks):
        table[i, :count] = torch.tensor(order[at:at + count], dtype=torch.int32)
        at += count
    table = table.cuda()
    starts = [n - m for n, m in zip(lengths, new)]
    positions = torch.cat([torch.arange(s, s + m) for s, m in zip(starts, new)]).int().cuda()
    token_item = torch.cat([torch.full((m,), i) for i, m in enumerate(new)]).int().cuda()
    n = sum(new)
    q = torch.randn(n, heads * dim, device="cuda") * 0.7
    want = torch.empty(n, heads * vdim, device="cuda")
    ops.capped_attention(want, q, k_pages, v_pages, table, positions, token_item, heads, kv_heads, dim, vdim, page_size, 0.4, cap)
    for window in (0, 21):
        plain_out = torch.empty_like(want)
        ops.capped_attention(plain_out, q, k_pages, v_pages, table, positions, token_item, heads, kv_heads, dim, vdim, page_size,
                             0.4, cap, window)
        got = torch.full_like(want, float("nan"))
        ops.capped_attention(got, q, k_pages, v_pages, table, positions, token_item, heads, kv_heads, dim, vdim, page_size, 0.4,
                             cap, window, tiled=True)
        torch.testing.assert_close(got, plain_out, rtol=2e-5, atol=2e-5)
    # the formula, for the last token of the second request
    row, item, p = new[0] + new[1] - 1, 1, lengths[1] - 1
    slots = [(int(table[item, j // page_size]), j % page_size) for j in range(p + 1)]
    for head in (0, heads - 1):
        g = head // (heads // kv_heads)
        keys = torch.stack([k_pages[a, b, g] for a, b in slots]).double()
        values = torch.stack([v_pages[a, b, g] for a, b in slots]).double()
        score = keys @ q[row, head * dim:(head + 1) * dim].double() * 0.4
        if cap:
            score = cap * torch.tanh(score / cap)
        expected = torch.softmax(score, 0) @ values
        torch.testing.assert_close(want[row, head * vdim:(head + 1) * vdim].double(), expected, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("heads, kv_heads, size, cap", [(4, 2, 64, 5.0), (6, 1, 128, 0.0), (3, 3, 32, 1.5)])
def test_single_tokens_over_split_keys_with_a_cap(heads, kv_heads, size, cap):
    """A step of single tokens in bfloat16: each token's keys in chunks over many blocks, with the cap
    on the scores, against the kernel with one block per (token, head)."""
    from mini_llm_b200.kernels import ops
    torch.manual_seed(size + heads)
    page_size, lengths = 16, [700, 1, 130, 64]
    blocks = [-(-n // page_size) for n in lengths]
    k_pages = torch.randn(sum(blocks) + 1, page_size, kv_heads, size, device="cuda").bfloat16()
    v_pages = torch.randn(sum(blocks) + 1, page_size, kv_heads, size, device="cuda").bfloat16()
    order = torch.randperm(sum(blocks)).tolist()
    table = torch.zeros(len(lengths), max(blocks), dtype=torch.int32)
    at = 0
    for i, count in enumerate(blocks):
        table[i, :count] = torch.tensor(order[at:at + count], dtype=torch.int32)
        at += count
    table = table.cuda()
    n = len(lengths)
    positions = dev([length - 1 for length in lengths], torch.int32)
    token_item = dev(list(range(n)), torch.int32)
    q = (torch.randn(n, heads * size, device="cuda") * 0.5).bfloat16()
    want = torch.empty(n, heads * size, device="cuda", dtype=torch.bfloat16)
    ops.capped_attention(want, q, k_pages, v_pages, table, positions, token_item, heads, kv_heads, size, size, page_size, 0.3, cap)
    chunk, reach = 64, table.shape[1] * page_size
    chunks = -(-reach // chunk)
    scratch = (torch.empty(n * heads * chunks * size, device="cuda"), torch.empty(n * heads * chunks * 2, device="cuda"),
               torch.zeros(n * heads, dtype=torch.int32, device="cuda"))
    got = torch.full_like(want, float("nan"))
    ops.split_attention(got, q, k_pages, v_pages, table, positions, token_item, heads, kv_heads, size, page_size, 0.3, 0, chunk,
                        chunks, *scratch, cap=cap)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    assert int(scratch[2].abs().max()) == 0


def test_rotation_and_cache_store():
    from mini_llm_b200.kernels import ops
    from mini_llm_b200.parts.rotary import rotary_frequencies
    rng = np.random.default_rng(5)
    heads, kv_heads, dim, vdim, page_size = 3, 1, 10, 6, 4
    rot = {"base": 300.0, "dims": 6, "scaling": sz.YARN}
    positions = np.array([0, 1, 2, 3, 4, 900, 901])
    token_item = np.array([0, 0, 0, 0, 0, 1, 1])
    table = np.full((2, 230), 0, dtype=np.int32)
    table[0, :2] = [3, 1]
    table[1, 225] = 2
    n = len(positions)
    rows = rng.normal(0, 1, (n, heads * dim + kv_heads * (dim + vdim)))
    qkv = dev(rows)
    k_pages = torch.zeros((4, page_size, kv_heads, dim), device="cuda")
    v_pages = torch.zeros((4, page_size, kv_heads, vdim), device="cuda")
    freqs, amplitude = rotary_frequencies(rot["base"], rot["dims"], rot["scaling"])
    ops.rotary_store(qkv, heads * dim, (heads + kv_heads) * dim, heads, kv_heads, dim, vdim, rot["dims"],
                     dev(freqs, torch.float64), amplitude, dev(positions, torch.int32), dev(token_item, torch.int32),
                     dev(table, torch.int32), page_size, k_pages, v_pages)
    q = plain.rotate_interleaved(rows[:, :heads * dim].reshape(n, heads, dim), positions, rot)
    k = plain.rotate_interleaved(rows[:, heads * dim:(heads + kv_heads) * dim].reshape(n, kv_heads, dim), positions, rot)
    got = qkv.cpu().numpy()
    np.testing.assert_allclose(got[:, :heads * dim], q.reshape(n, -1), atol=3e-6)
    np.testing.assert_allclose(got[:, heads * dim:(heads + kv_heads) * dim], k.reshape(n, -1), atol=3e-6)
    for t in range(n):
        page = table[token_item[t], positions[t] // page_size]
        np.testing.assert_allclose(k_pages[page, positions[t] % page_size].cpu().numpy(), k[t], atol=3e-6)
        np.testing.assert_allclose(v_pages[page, positions[t] % page_size].cpu().numpy().reshape(-1),
                                   rows[t, (heads + kv_heads) * dim:], atol=1e-7)


def test_router_and_expert_kernels():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(6)
    width, experts, top, inner, shared_inner, n = 40, 6, 3, 12, 20, 9
    x = rng.normal(0, 1, (n, width))
    w = {"m.router": rng.normal(0, 0.5, (experts, width)), "m.shared.sg": rng.normal(0, 0.3, (1, width))}
    for name, size in [(f"e{e}", inner) for e in range(experts)] + [("shared", shared_inner)]:
        w[f"m.{name}.gate"], w[f"m.{name}.up"] = rng.normal(0, 0.3, (size, width)), rng.normal(0, 0.3, (size, width))
        w[f"m.{name}.down"] = rng.normal(0, 0.3, (width, size))
    expected = plain.routed_experts(x, {"router": {"experts": experts, "top": top}, "shared": {"ff": shared_inner}}, w, "m")
    held = {name: dev(values) for name, values in w.items()}
    names = [f"e{e}" for e in range(experts)] + ["shared"]
    table = lambda which: torch.tensor([held[f"m.{name}.{which}"].data_ptr() for name in names], dtype=torch.int64, device="cuda")
    pairs = top + 1
    choice = torch.zeros(n * pairs, dtype=torch.int32, device="cuda")
    in_weight, out_weight = torch.zeros(n * pairs, device="cuda"), torch.zeros(n * pairs, device="cuda")
    ops.route(dev(x), held["m.router"], held["m.shared.sg"], top, choice, in_weight, out_weight)
    scores = plain.sigmoid(x @ w["m.router"].T)
    for t in range(n):
        assert choice[t * pairs:t * pairs + top].tolist() == np.argsort(-scores[t], kind="stable")[:top].tolist()
        assert int(choice[t * pairs + top]) == experts
    hidden = torch.ones((n, width), device="cuda")
    act = torch.empty((n * pairs, shared_inner), device="cuda")
    down_all = torch.cat([held[f"m.{name}.down"] for name in names], dim=1).contiguous()        # side by side, rows 92 apart
    starts = [e * inner for e in range(experts)] + [experts * inner]
    down_of = torch.tensor([down_all.data_ptr() + 4 * start for start in starts], dtype=torch.int64, device="cuda")
    ops.experts(hidden, act, dev(x), choice, in_weight, out_weight, table("gate"), table("up"), down_of,
                dev([inner] * experts + [shared_inner], torch.int32), shared_inner, pairs, ld_down=down_all.shape[1])
    np.testing.assert_allclose(hidden.cpu().numpy() - 1.0, expected, atol=2e-5)
    # the same through the products over all experts: gates and ups of every expert, unchosen ones weighed 0
    up_all = torch.cat([held[f"m.{name}.{which}"] for which in ("gate", "up") for name in names])
    gu = dev(x) @ up_all.T
    combined = torch.empty((n, down_all.shape[1]), device="cuda")
    ops.expert_combine(combined, gu.contiguous(), choice, in_weight, out_weight, experts, inner, top, pairs)
    np.testing.assert_allclose((combined @ down_all.T).cpu().numpy(), expected, atol=2e-5)
