"""Fuvolix on the device against the plain implementation (``plain_fuvolix``, float64).

Every test makes its own small configuration and random weights.  32-bit runs must agree within
1e-4; bfloat16 runs within the bound the other models' tests use.  The schedules cut the same
requests in different ways: a request's logits must not depend on the cut, on the rest of the
batch, or on which pages and slots it got."""

import numpy as np
import pytest
import torch

import fuvolix_helpers as fx
import plain_fuvolix as plain
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
        expected = fx.plain_logits(folder, tokens)
        worst = np.abs(got[name] - expected).max(axis=1)
        assert worst.max() <= atol, f"request {name}: first wrong token {int(np.argmax(worst > atol))} of {len(tokens)}, off by {worst.max():.2e}"
    engine.cache.check()


# ---- each mechanism alone ----------------------------------------------------------------------

@pytest.mark.parametrize("layer", [
    fx.latent(), fx.latent(ff=56), fx.latent(heads=1, dim=8, rot_dim=4, vdim=8, kv_rank=8, dims=0),
    fx.latent(heads=2, dim=24, rot_dim=24, vdim=8, kv_rank=136, dims=10),
    fx.mlstm(), fx.mlstm(heads=1, dim=4, vdim=70, gate_cap=2.0, ff=32),
    fx.lightning(), fx.lightning(heads=1, dim=40, vdim=33, decay=[1.0]),
], ids=["latent", "latent_ff", "latent_one_head_no_rotation", "latent_wide_rank_part_rotated", "mlstm", "mlstm_one_head",
        "lightning", "lightning_no_decay"])
def test_one_layer_of_each_mixer(tmp_path, layer):
    folder = fx.make_model(str(tmp_path / "m"), fx.config([layer]), seed=3, matrix_scale=3.0)
    engine = engine_for(folder)
    requests = {"a": random_tokens(1, 37, 211), "b": random_tokens(2, 1, 211), "c": random_tokens(3, 2, 211)}
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_portions(requests))


def test_residual_stream_after_every_layer(tmp_path):
    from mini_llm_b200.engine import StepEntry
    folder = fx.make_model(str(tmp_path / "m"), fx.full_stack(), seed=5, matrix_scale=2.0)
    engine = engine_for(folder)
    tokens = random_tokens(4, 29, 211)
    streams = []
    fx.plain_logits(folder, tokens, streams)
    slot = engine.open_request()
    engine.step([StepEntry(slot, tokens, [28])], dump_hidden=True)
    assert len(engine.hidden_dump) == len(streams) + 1
    for index, expected in enumerate(streams):
        np.testing.assert_allclose(engine.hidden_dump[index + 1].cpu().numpy(), expected, rtol=0,
                                   atol=1e-4 * np.abs(expected).max(), err_msg=f"after layer {index}")
    engine.close_request(slot)


# ---- the same tokens, cut differently -----------------------------------------------------------

@pytest.mark.parametrize("kwargs", [dict(), dict(taps=1, groups=1), dict(taps=6, groups=8), dict(taps=2, groups=32)],
                         ids=["taps3", "no_taps_one_group", "six_taps", "two_taps_groups_of_three"])
def test_prompt_against_token_by_token_and_portions(tmp_path, kwargs):
    folder = fx.make_model(str(tmp_path / "m"), fx.full_stack(**kwargs), seed=7, bend=fx.sharpen(6.0), matrix_scale=2.0)
    engine = engine_for(folder)
    requests = {"a": random_tokens(11, 45, 211), "b": random_tokens(12, 7, 211)}
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=45))        # every token alone, from the first
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=5))
    check(engine, folder, requests, schedule_portions(requests))
    check(engine, folder, requests, schedule_portions(requests, sizes=(2, 2, 3, 2, 17)))
    if "taps" not in kwargs:
        assert engine.step_kinds["replayed"] > 0          # steps of one shape were replayed from a captured graph


def test_mixed_batches_and_reuse_of_pages_and_slots(tmp_path):
    """Six requests through three slots and a page pool that holds less than their sum: pages
    and slots are given back and used again (and poisoned in between), portions run beside
    single tokens; every request must come out as it does alone."""
    folder = fx.make_model(str(tmp_path / "m"), fx.full_stack(), seed=9, bend=fx.sharpen(6.0), matrix_scale=2.0)
    lengths = {"a": 61, "b": 9, "c": 33, "d": 2, "e": 40, "f": 18}
    requests = {name: random_tokens(20 + i, n, 211) for i, (name, n) in enumerate(lengths.items())}
    prompts = {"a": 40, "b": 9, "c": 20, "d": 1, "e": 40, "f": 3}
    engine = engine_for(folder, max_requests=3, cache_tokens=160, debug_poison=True)
    check(engine, folder, requests, schedule_mixed(requests, prompts, max_live=3))
    check(engine, folder, requests, schedule_mixed(requests, prompts, max_live=2, portion_sizes=(2, 11, 3)))
    assert not any(engine.cache.pages_in_use()) and engine.cache.free_slots == 3


def test_a_far_key_decides(tmp_path):
    """One early token's key is made to match the last query, and its value to stand out: the
    logits then hang on that single far key (behind many page borders), in a prompt and when the
    last token is decoded alone."""
    raw = fx.config([fx.latent(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16, scale=1.0, dims=4)], vocab=64)
    def bend(t):
        # only token 5 (and, with the other sign, token 9) has anything in the first eight channels;
        # the first latent entry reads them, the first query entry of head 0 reads them too, and
        # head 0's first key entry is that latent entry: token 9's query finds token 5's key
        t["embed"][:, :8] = 0.0
        t["embed"][5, :8] = 2.0
        t["embed"][9, :8] = -2.0
        t["l0.mix.dkv"][0] = 0.0
        t["l0.mix.dkv"][0, :8] = 4.0
        t["l0.mix.q"][0] = 0.0
        t["l0.mix.q"][0, :8] = -0.5
        t["l0.mix.uk"][0] = 0.0
        t["l0.mix.uk"][0, 0] = 1.0
    folder = fx.make_model(str(tmp_path / "m"), raw, seed=13, bend=bend, matrix_scale=2.0)
    rng = np.random.default_rng(0)
    base = [int(t) for t in rng.integers(10, 64, 300)]
    base[-1] = 9
    with_key, without = list(base), list(base)
    with_key[3] = 5
    assert np.abs(fx.plain_logits(folder, with_key)[-1] - fx.plain_logits(folder, without)[-1]).max() > 0.1
    engine = engine_for(folder)
    for tokens in (with_key, without):
        requests = {"r": tokens}
        check(engine, folder, requests, schedule_whole(requests))
        check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=3))
        check(engine, folder, requests, schedule_portions(requests, sizes=(8, 7, 9, 64, 2)))


def test_long_decoding_with_gates_that_move_the_maximum(tmp_path):
    """A hundred and fifty tokens one by one; the gate biases are bent so that the running
    maximum of the gated memory climbs, falls and is overtaken by the input gate."""
    raw = fx.config([fx.mlstm(heads=2, dim=8, vdim=8, gate_cap=6.0), fx.lightning(heads=2, dim=8, vdim=8, decay=[0.999, 0.3]),
                     fx.mlstm(heads=1, dim=16, vdim=8, gate_cap=20.0, ff=24)], width=32, groups=2, vocab=97)
    def bend(t):
        t["l0.mix.i.b"][:] = [3.0, -4.0]
        t["l0.mix.f.b"][:] = [-3.0, 5.0]
        t["l0.mix.i"] *= 40.0
        t["l2.mix.f"] *= 40.0
        t["l2.mix.i.b"][:] = 8.0
    folder = fx.make_model(str(tmp_path / "m"), raw, seed=17, bend=bend, matrix_scale=2.0)
    engine = engine_for(folder)
    requests = {"long": random_tokens(31, 151, 97)}
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=150))
    check(engine, folder, requests, schedule_whole(requests))


def test_bfloat16_follows_within_its_rounding(tmp_path):
    folder = fx.make_model(str(tmp_path / "m"), fx.full_stack(width=128, groups=4), seed=19, matrix_scale=2.0)
    engine = engine_for(folder, dtype="bfloat16")
    requests = {"a": random_tokens(41, 140, 211), "b": random_tokens(42, 12, 211), "c": random_tokens(43, 70, 211)}
    bound = max(bf16_atol(fx.plain_logits(folder, tokens)) for tokens in requests.values())
    check(engine, folder, requests, schedule_whole(requests), atol=bound)
    check(engine, folder, requests, schedule_mixed(requests, {"a": 100, "b": 6, "c": 64}, max_live=3), atol=bound)
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=10), atol=bound)


def test_greedy_generation_through_the_scheduler(tmp_path):
    from mini_llm_b200.generate import generate
    folder = fx.make_model(str(tmp_path / "m"), fx.full_stack(), seed=23, matrix_scale=3.0)
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

def test_grouped_rms_norm_kernel():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(1)
    x = rng.normal(0, 2, (9, 120))
    gain = rng.uniform(0.5, 1.5, 120)
    xd = torch.tensor(x, dtype=torch.float32, device="cuda")
    gd = torch.tensor(gain, dtype=torch.float32, device="cuda")
    for groups in (1, 3, 8, 120):
        out = torch.empty_like(xd)
        ops.grouped_rms_norm(out, xd, gd, groups, 1e-3)
        np.testing.assert_allclose(out.cpu().numpy(), plain.grouped_rms_norm(x, gain, groups, 1e-3), atol=2e-6)
    base = rng.normal(0, 1, (9, 120))
    summed = torch.tensor(base, dtype=torch.float32, device="cuda")
    ops.grouped_rms_norm(summed, xd, gd, 4, 1e-5, add=True)
    np.testing.assert_allclose(summed.cpu().numpy(), base + plain.grouped_rms_norm(x, gain, 4, 1e-5), atol=2e-6)
    gate = rng.normal(0, 2, (9, 120))
    out = torch.empty_like(xd)
    ops.grouped_rms_norm(out, xd, gd, 2, 1e-5, gate=torch.tensor(gate, dtype=torch.float32, device="cuda"))
    np.testing.assert_allclose(out.cpu().numpy(), plain.grouped_rms_norm(x, gain, 2, 1e-5) * plain.sigmoid(gate), atol=2e-6)


def test_causal_taps_kernel_over_cuts():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(2)
    width, taps = 20, 4
    h = {0: rng.normal(0, 1, (11, width)), 1: rng.normal(0, 1, (5, width))}
    w = rng.normal(0, 0.5, (width, taps))
    expected = {i: plain.causal_taps(h[i], w) for i in h}
    dev = lambda a, dt=torch.float32: torch.tensor(np.asarray(a), dtype=dt, device="cuda")
    state = torch.zeros((3, taps - 1, width), dtype=torch.float32, device="cuda")
    got = {0: [], 1: []}
    done = {0: 0, 1: 0}
    # request 0 lives in slot 2, request 1 in slot 0; portions of 1, 2 and more tokens, in one batch
    for cut in ({0: 1, 1: 2}, {0: 2, 1: 1}, {0: 5}, {1: 2, 0: 3}):
        rows, positions, token_item, slots, starts, offsets, counts = [], [], [], [], [], [], []
        for item, (request, n) in enumerate(cut.items()):
            offsets.append(len(positions))
            rows.append(h[request][done[request]:done[request] + n])
            positions += list(range(done[request], done[request] + n))
            token_item += [item] * n
            slots.append(2 if request == 0 else 0)
            starts.append(done[request])
            counts.append(n)
        x = dev(np.concatenate(rows))
        out = torch.empty_like(x)
        ops.causal_taps(out, x, dev(w), state, dev(positions, torch.int32), dev(token_item, torch.int32),
                        dev(slots, torch.int32), dev(starts, torch.int32), dev(offsets, torch.int32), dev(counts, torch.int32))
        for item, (request, n) in enumerate(cut.items()):
            got[request].append(out[offsets[item]:offsets[item] + n].cpu().numpy())
            done[request] += n
    for request in (0, 1):
        np.testing.assert_allclose(np.concatenate(got[request]), expected[request][:done[request]], atol=2e-6)


def test_memory_scan_kernel_carries_its_state():
    """Both recurrences, a sequence cut in three, against the token-by-token formulas."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(3)
    heads, dim, vdim, n = 2, 12, 37, 100
    q, k = rng.normal(0, 1, (n, heads * dim)), rng.normal(0, 1, (n, heads * dim))
    v = rng.normal(0, 1, (n, heads * vdim))
    gates = rng.normal(0, 6, (n, 2 * heads))
    bias = rng.normal(0, 1, 2 * heads)
    cap, decay = 5.0, [0.9, 0.4]
    dev = lambda a, dt=torch.float32: torch.tensor(np.asarray(a), dtype=dt, device="cuda")

    expected_gated = np.zeros((n, heads, vdim))
    expected_fixed = np.zeros((n, heads, vdim))
    for head in range(heads):
        S, nv, m = np.zeros((dim, vdim)), np.zeros(dim), 0.0
        F = np.zeros((dim, vdim))
        for t in range(n):
            qt, kt = q[t, head * dim:(head + 1) * dim], k[t, head * dim:(head + 1) * dim]
            vt = v[t, head * vdim:(head + 1) * vdim]
            li = cap * np.tanh((gates[t, head] + bias[head]) / cap)
            lf = plain.log_sigmoid(cap * np.tanh((gates[t, heads + head] + bias[heads + head]) / cap))
            m_new = max(lf + m, li)
            a, b = np.exp(lf + m - m_new), np.exp(li - m_new)
            S, nv, m = a * S + b * np.outer(kt, vt), a * nv + b * kt, m_new
            expected_gated[t, head] = S.T @ (qt * 0.5) / (max(abs(nv @ (qt * 0.5)), np.exp(-m)) + 1e-6)
            F = decay[head] * F + np.outer(plain.silu(kt), plain.silu(vt))
            expected_fixed[t, head] = F.T @ plain.silu(qt)
    for gated, chunked in ((True, False), (False, False), (True, True), (False, True), (True, "passes"), (False, "passes")):
        state = torch.zeros((2, ops.memory_state_floats(heads, dim, vdim, gated)), dtype=torch.float32, device="cuda")
        out = torch.empty((n, heads * vdim), dtype=torch.float32, device="cuda")
        for first, count in ((0, 1), (1, 9), (10, 13), (23, 32), (55, 45)):
            how = (dict(gates=dev(gates), gate_bias=dev(bias), gate_cap=cap, q_scale=0.5) if gated
                   else dict(decay=dev(decay), silu=True))
            # entry 0 is another request with no tokens in this step; entry 1 is ours, in slot 1
            passes = None
            if chunked == "passes":
                passes = [torch.full((floats,), float("nan"), device="cuda") for floats in ops.memory_passes_scratch(n, 2, heads, dim, vdim)]
            ops.memory_scan(out, dev(q), dev(k), dev(v), state, dev([0, 1], torch.int32), dev([0, first], torch.int32),
                            dev([0, count], torch.int32), heads, dim, vdim, chunked=chunked is True, passes=passes, **how)
        expected = (expected_gated if gated else expected_fixed).reshape(n, heads * vdim)
        # (the gates here are extreme, so n . q nearly cancels now and then, and the quotient carries the
        # sums' rounding ten times over; the chunked kernel adds in another order than the formulas above)
        np.testing.assert_allclose(out.cpu().numpy(), expected, rtol=5e-4 if chunked else 5e-5, atol=2e-5,
                                   err_msg=f"gated {gated}, chunked {chunked}")
        assert float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("heads, rank, rot", [(3, 40, 8), (1, 8, 4), (6, 128, 32), (16, 264, 24), (40, 16, 0)])
def test_latent_attention_in_tiles_against_the_plain_kernel(heads, rank, rot):
    """Prompt portions through the work list, and single tokens with their keys in parts: the tiled
    kernel must give what the kernel with one block per (token, head) gives, on 32-bit pages."""
    from mini_llm_b200.kernels import ops
    torch.manual_seed(heads * 1000 + rank)
    page_size, row = 8, rank + rot
    lengths, new = [150, 9, 77], [150, 3, 40]                 # cached + new tokens; tokens of this step
    blocks = [-(-n // page_size) for n in lengths]
    pages = torch.randn(sum(blocks) + 1, page_size, 1, row, device="cuda")
    order = torch.randperm(sum(blocks)).tolist()              # pages scattered over the pool
    table = torch.zeros(3, max(blocks), dtype=torch.int32)
    at = 0
    for i, count in enumerate(blocks):
        table[i, :count] = torch.tensor(order[at:at + count], dtype=torch.int32)
        at += count
    table = table.cuda()
    offsets = [0, new[0], new[0] + new[1]]
    starts = [n - m for n, m in zip(lengths, new)]
    positions = torch.cat([torch.arange(s, s + m) for s, m in zip(starts, new)]).int().cuda()
    token_item = torch.cat([torch.full((m,), i) for i, m in enumerate(new)]).int().cuda()
    n = sum(new)
    q_eff = torch.randn(n, heads * row, device="cuda") * 0.7
    want = torch.empty(n, heads * rank, device="cuda")
    ops.latent_attention_plain(want, q_eff, pages, table, positions, token_item, heads, rank, rot, page_size, 0.4)
    tiles, _, _ = ops.attention_tiles(offsets, new, starts)          # few tiles: the long one comes in parts, which are skipped
    got = torch.full_like(want, float("nan"))
    ops.latent_attention_tiled(got, q_eff, pages, table, positions, token_item, heads, rank, rot, page_size, 0.4,
                               tiles=torch.tensor(tiles, dtype=torch.int32, device="cuda"), n_tiles=len(tiles))
    torch.testing.assert_close(got, want, rtol=2e-5, atol=2e-5)
    # single tokens: the last token of each request, keys in 1, 3 and 5 parts
    last = torch.tensor([offsets[i] + new[i] - 1 for i in range(3)], device="cuda")
    for parts in (1, 3, 5):
        scratch = (torch.empty(3 * heads * parts * rank, device="cuda"), torch.empty(3 * heads * parts * 2, device="cuda"))
        got = torch.full((3, heads * rank), float("nan"), device="cuda")
        ops.latent_attention_tiled(got, q_eff[last].contiguous(), pages, table, positions[last].contiguous(),
                                   token_item[last].contiguous(), heads, rank, rot, page_size, 0.4, parts=parts,
                                   scratch=scratch)
        torch.testing.assert_close(got, want[last], rtol=2e-5, atol=2e-5)


def test_bfloat16_with_sizes_no_fast_kernel_takes(tmp_path):
    """A width that is no multiple of 8, a latent that is no multiple of 8, key sizes of 5 and 6: every
    product, the attention and the memories fall back to kernels that take any size, in bfloat16
    too, for prompts, portions and single tokens."""
    raw = fx.config([fx.latent(heads=3, dim=10, rot_dim=6, vdim=14, kv_rank=22, ff=52), fx.mlstm(heads=2, dim=6, vdim=10),
                     fx.lightning(heads=3, dim=5, vdim=7, ff=36), fx.latent(heads=5, dim=4, rot_dim=2, vdim=6, kv_rank=13, dims=2)],
                    width=100, groups=5, vocab=203, taps=5)
    folder = fx.make_model(str(tmp_path / "m"), raw, seed=29, matrix_scale=2.0)
    requests = {"a": random_tokens(61, 150, 203), "b": random_tokens(62, 3, 203), "c": random_tokens(63, 40, 203)}
    bound = max(bf16_atol(fx.plain_logits(folder, tokens)) for tokens in requests.values())
    engine = engine_for(folder, dtype="bfloat16")
    check(engine, folder, requests, schedule_whole(requests), atol=bound)
    check(engine, folder, requests, schedule_mixed(requests, {"a": 130, "b": 2, "c": 33}, max_live=3), atol=bound)
    chosen = {kernel for key, kernel in engine.kernels.choices.items() if key[0] in ("latent_attention", "head_linear", "linear")}
    assert chosen == {"latent_attention_plain", "head_linear_plain", "linear_plain"}
    engine32 = engine_for(folder)
    check(engine32, folder, requests, schedule_portions(requests))
