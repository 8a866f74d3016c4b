"""The Nodopel design in the engine against the plain implementation: every kernel alone, whole models
under every way of cutting requests into steps, pages and slots that are used again, and greedy
generation through the engine's own entry point.  float32 runs are compared tightly, bfloat16 runs as a
fraction of the largest logit."""

from __future__ import annotations

import math

import pytest
import torch

import helpers
import nodopel_configs
import plain_nodopel as plain

pytestmark = pytest.mark.gpu

CONFIGS, LENGTHS = nodopel_configs.CONFIGS, nodopel_configs.LENGTHS
F32_REL, BF16_REL = 3e-5, 0.06


def steady_choice(weights, raw):
    """Corrections two apart from expert to expert, in a shuffled order of their own in every layer: a softmax
    score lies between 0 and 1, so the choice of experts never hangs on a close call between two scores, while
    the weights of the chosen still differ from token to token."""
    generator = torch.Generator().manual_seed(77)
    for name, tensor in weights.items():
        if name.endswith(".correction"):
            levels = 2.0 * torch.randperm(tensor.shape[0], generator=generator).float()
            weights[name] = (levels - levels.mean().round()).to(tensor.dtype)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """Stored in bfloat16: both run modes and the plain implementation then read the same numbers.  The
    float32 runs route as the random weights say; the bfloat16 runs get models whose choice of experts is
    steady (the rounding of the stream would otherwise turn a close call the other way now and then, which
    changes a row by far more than rounding)."""
    made = {}
    for i, (name, (raw, _)) in enumerate(CONFIGS.items()):
        made[name, "float32"] = helpers.make_model_folder(tmp_path_factory.mktemp("nodopel"), raw, seed=31 + i,
                                                          dtype=torch.bfloat16)
        made[name, "bfloat16"] = helpers.make_model_folder(tmp_path_factory.mktemp("nodopel_steady"), raw, seed=31 + i,
                                                           dtype=torch.bfloat16, special=steady_choice)
    return made


def load_plain(folder, raw):
    from safetensors import safe_open
    weights = {}
    with safe_open(str(folder / "model.safetensors"), "pt") as handle:
        for key in handle.keys():
            weights[key] = handle.get_tensor(key).double()
    return plain.PlainNodopel(raw, weights)


@pytest.fixture(scope="module")
def references(folders):
    out = {}
    for (name, dtype), folder in folders.items():
        raw = CONFIGS[name][0]
        model = load_plain(folder, raw)
        sequences = {rid: helpers.random_tokens(raw["vocab"], n, seed=sum(map(ord, name + rid)))
                     for rid, n in LENGTHS[name].items()}
        out[name, dtype] = (sequences, {rid: model.run(rid, tokens).float() for rid, tokens in sequences.items()})
    return out


def make_runner(folder, dtype, page_size, num_pages, max_requests=4):
    from vllm_from_scratch_b200 import ModelRunner
    return ModelRunner.from_folder(folder, dtype, page_size, num_pages, max_requests, device="cuda")


def compare(results, expected, dtype, what):
    bound_rel = F32_REL if dtype == "float32" else BF16_REL
    worst = 0.0
    for rid, logits in results.items():
        reference = expected[rid]
        assert logits.shape == reference.shape, (what, rid, logits.shape, reference.shape)
        diff = (logits - reference).abs()
        bound = bound_rel * float(reference.abs().max())
        if not float(diff.max()) <= bound:
            position = int((~diff.max(dim=1).values.le(bound)).nonzero()[0])
            raise AssertionError(f"{what}: request {rid!r} first differs at position {position} "
                                 f"(max |diff| there {float(diff[position].max()):.3e}, bound {bound:.3e})")
        worst = max(worst, float(diff.max()) / float(reference.abs().max()))
    print(f"{what}: worst difference as a fraction of the largest logit {worst:.3e}")


CUTS = {
    "whole": lambda lengths: helpers.cut_whole(lengths),
    "tail": lambda lengths: helpers.cut_tail_one_by_one(lengths, 40),
    "portions": lambda lengths: helpers.cut_changing_portions(lengths, seed=1),
    "one_by_one": lambda lengths: [[(rid, 1)] for rid, n in lengths.items() if n <= 70 for _ in range(n)],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_each_request_alone(folders, references, name, cut, dtype):
    """Whole prompts, prompts whose last 40 tokens are decoded one by one (windows pass over decoded tokens),
    portions of changing sizes down to two tokens, and whole sequences decoded token by token."""
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name, dtype]
    steps = CUTS[cut](LENGTHS[name])
    used = {rid for step in steps for rid, _ in step}
    longest = max(LENGTHS[name].values())
    runner = make_runner(folders[name, dtype], dtype, page_size, -(-longest // page_size) + 1)
    results = helpers.run_schedule(runner, {rid: sequences[rid] for rid in used}, steps)
    compare(results, expected, dtype, f"{name}/{cut}/{dtype}")
    runner.check_device()
    assert runner.manager.stats()["requests"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [0, 1])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_few_pages_and_slots(folders, references, name, seed, dtype):
    """Up to three live requests in three slots, portions beside single tokens, requests left out of steps,
    and a pool so small that the pages of a finished request are handed out again at once (windowed groups
    also give pages back while a request runs, all but those of the first positions that stay visible)."""
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name, dtype]
    steps = helpers.cut_mixed(LENGTHS[name], seed=seed, live=3, sizes=(2, 3, 5, 8, 13, 16, 21, 33, 70))
    pages = sum(sorted((-(-n // page_size) for n in LENGTHS[name].values()), reverse=True)[:3])
    runner = make_runner(folders[name, dtype], dtype, page_size, pages, max_requests=3)
    results = helpers.run_schedule(runner, sequences, steps)
    compare(results, expected, dtype, f"{name}/mixed{seed}/{dtype}")
    assert runner.manager.stats()["requests"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, references, dtype):
    """A short prompt and 220 tokens decoded one by one: every window moves over decoded tokens only, the
    windowed groups give back the pages behind them and keep those of the first positions."""
    raw, page_size = CONFIGS["D"]
    sequences, expected = references["D", dtype]
    runner = make_runner(folders["D", dtype], dtype, page_size, 14)
    steps = [[("g", 10)]] + [[("g", 1)] for _ in range(220)]
    results = helpers.run_schedule(runner, {"g": sequences["g"]}, steps)
    compare(results, expected, dtype, "D/long decode")
    windowed = [group for group, window in enumerate(runner.manager.group_windows) if window is not None]
    assert windowed and all(runner.manager.num_free_pages(group) == 14 for group in windowed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_engine(folders, name, dtype):
    """``LLM.generate`` (scheduler, token budget, graph replay of decode steps, steps queued ahead) gives
    the tokens that the plain implementation's argmax gives, for prompts of unequal lengths that are cut by
    the token budget and run side by side."""
    import vllm_from_scratch_b200 as engine
    raw, page_size = CONFIGS[name]
    model = load_plain(folders[name, dtype], raw)
    prompts = [helpers.random_tokens(raw["vocab"], n, seed=40 + n) for n in (5, 37, 1, 60)]
    new_tokens = 12
    llm = engine.LLM(str(folders[name, dtype]), dtype=dtype, max_model_len=128, block_size=page_size, num_gpu_blocks=40,
                     max_num_seqs=3, max_num_batched_tokens=24)
    outputs = llm.generate(prompts, engine.SamplingParams(max_tokens=new_tokens, temperature=0.0, ignore_eos=True))
    assert llm.engine.decode_graphs is not None and llm.engine.decode_graphs.replays > 0
    for number, (prompt, output) in enumerate(zip(prompts, outputs)):
        logits = model.run(number, prompt)
        for index, token in enumerate(output.token_ids):
            row = logits[-1]
            best = int(row.argmax())
            if token != best:
                # bfloat16 may swap two tokens that the plain implementation puts within its noise
                gap = float(row[best] - row[token]) / float(row.abs().max())
                assert dtype == "bfloat16" and gap < 0.03, (index, token, best, gap)
            logits = model.run(number, [token])
        assert len(output.token_ids) == new_tokens
    llm.engine.shutdown()


def test_preempted_requests_are_computed_again(folders):
    """A pool too small for all requests at once: some are preempted, lose their pages (those of the first
    positions too), and are computed again from their first token; every request still ends with the tokens
    it gets from a large pool."""
    import vllm_from_scratch_b200 as engine
    raw, page_size = CONFIGS["A"]
    prompts = [helpers.random_tokens(raw["vocab"], n, seed=70 + i) for i, n in enumerate([30, 41, 18, 25])]
    params = engine.SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    results = {}
    for label, blocks in (("large", 64), ("small", 8)):
        llm = engine.LLM(str(folders["A", "float32"]), dtype="float32", max_model_len=128, block_size=page_size,
                         num_gpu_blocks=blocks, max_num_seqs=4, max_num_batched_tokens=64)
        results[label] = llm.generate(prompts, params)
        if label == "small":
            assert llm.engine.scheduler.num_preemptions > 0, "the small pool was meant to run out"
        llm.engine.runner.manager.check_invariants()
        llm.engine.shutdown()
    for big, small in zip(results["large"], results["small"]):
        assert big.token_ids == small.token_ids


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(folders, references, tmp_path, dtype):
    """``bin/trace_run`` in a process of its own: a mixed schedule of up to four live requests over a pool
    of 4 x 128 positions, logits of every place written step by step."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np
    root = Path(__file__).resolve().parent.parent
    name = "A"
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name, dtype]
    lengths = {rid: min(n, 128) for rid, n in LENGTHS[name].items()}
    sequences = {rid: tokens[:lengths[rid]] for rid, tokens in sequences.items()}
    steps = helpers.cut_mixed(lengths, seed=5, live=4)
    lines = helpers.schedule_to_trace(sequences, steps)
    out = tmp_path / "out"
    process = subprocess.run(
        [sys.executable, str(root / "bin" / "trace_run"), "--model", str(folders[name, dtype]), "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(4 * 128)],
        input="\n".join(json.dumps(line) for line in lines) + "\n", capture_output=True, text=True,
        timeout=900, env={**os.environ, "PYTHONPATH": ""})
    assert process.returncode == 0, process.stderr[-3000:]
    assert [l for l in process.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(lines))]
    results: dict = {rid: [] for rid in sequences}
    for line in lines:
        data = torch.from_numpy(np.fromfile(out / f"{line['step']}.f32", dtype="<f4").reshape(-1, raw["vocab"]).copy())
        at = 0
        for entry in line["entries"]:
            results[entry["id"]].append(data[at:at + len(entry["tokens"])])
            at += len(entry["tokens"])
        assert at == data.shape[0]
    compare({rid: torch.cat(rows) for rid, rows in results.items()},
            {rid: expected[rid][:lengths[rid]] for rid in sequences}, dtype, f"replay program/{dtype}")


# ------------------------------------------------------------------- kernels alone
def dev(tensor, dtype=None):
    return tensor.to("cuda", dtype) if dtype is not None else tensor.to("cuda")


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


def rounded(tensor, dtype):
    """What the engine reads of a tensor made in float64: its rounding to the run dtype."""
    return tensor.to(dtype).double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 64), (2, 50), (3, 352), (5, 37), (8, 1024), (11, 72), (16, 128)])
def test_streams_between_two_sublayers(dtype, shape):
    """Every stream set to the embedding's rows; the update by a sublayer's rows with the read and norm of the
    next; the plain sum for the last norm, on a few rows only and without touching the streams."""
    from vllm_from_scratch_b200.kernels import streams as kernels_streams
    count, hidden = shape
    tokens, eps = 19, 1e-5
    g = torch.Generator().manual_seed(count * 1000 + hidden)
    fresh = torch.randn(tokens, hidden, generator=g)
    w_in, w_out = torch.randn(count, generator=g), torch.randn(count, generator=g)
    mix = torch.eye(count) + 0.3 * torch.randn(count, count, generator=g)
    norm_w = 1.0 + 0.2 * torch.randn(hidden, generator=g)
    y = torch.randn(tokens, hidden, generator=g).to(dtype)
    X = torch.empty(tokens, count, hidden, device="cuda")
    normed = torch.empty(tokens, hidden, dtype=dtype, device="cuda")
    tolerance = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)

    kernels_streams.stream_mix_norm(X, fresh=dev(fresh), in_weights=dev(w_in), norm_weight=dev(norm_w), eps=eps,
                                    normed=normed)
    plain_X = [fresh[t].double()[None, :].repeat(count, 1) for t in range(tokens)]
    assert torch.equal(X.cpu(), torch.stack(plain_X).float())
    want = torch.stack([plain.rms(plain.streams_read(x, w_in.double()), eps) * norm_w.double() for x in plain_X])
    assert torch.allclose(normed.cpu().double(), want, **tolerance)

    kernels_streams.stream_mix_norm(X, rows_in=dev(y), mix=dev(mix), out_weights=dev(w_out), in_weights=dev(w_in),
                                    norm_weight=dev(norm_w), eps=eps, normed=normed)
    plain_X = [plain.streams_write(x, mix.double(), w_out.double(), y[t].double()) for t, x in enumerate(plain_X)]
    assert torch.allclose(X.cpu().double(), torch.stack(plain_X), rtol=1e-6, atol=1e-6)
    want = torch.stack([plain.rms(plain.streams_read(x, w_in.double()), eps) * norm_w.double() for x in plain_X])
    assert torch.allclose(normed.cpu().double(), want, **tolerance)

    # the model's last norm: the update is still to come, only some rows are wanted, the streams stay
    before = X.clone()
    rows = [17, 0, 5]
    some = torch.empty(len(rows), hidden, dtype=dtype, device="cuda")
    kernels_streams.stream_mix_norm(X, rows_in=dev(y), mix=dev(mix), out_weights=dev(w_out), norm_weight=dev(norm_w),
                                    eps=eps, normed=some, rows=i32(rows))
    assert torch.equal(X, before)
    want = torch.stack([plain.rms(plain.streams_write(plain_X[t], mix.double(), w_out.double(), y[t].double()).sum(0), eps)
                        * norm_w.double() for t in rows])
    assert torch.allclose(some.cpu().double(), want, **tolerance)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(5, 1, 48, 80, 32), (3, 3, 10, 6, 6), (2, 1, 64, 128, 0), (6, 2, 16, 24, 16), (1, 1, 128, 64, 2),
                                   (2, 2, 20, 12, 8), (2, 1, 6, 10, 4), (3, 1, 32, 16, 32)])
def test_bias_rotation_and_pages(dtype, shape):
    """Biases, the rotation of the first numbers of every map of every head at far positions, keys and
    values into scattered slots; a token without a slot stores nothing."""
    from vllm_from_scratch_b200.kernels import differential
    H, G, d, dv, rotary = shape
    tokens, page, pages = 7, 4, 6
    g = torch.Generator().manual_seed(d + dv)
    width = (H + G) * 2 * d + G * dv
    qkv = torch.randn(tokens, width, generator=g).to(dtype)
    bias = torch.randn(width, generator=g)
    positions = [0, 1, 5, 1000, 77777, 31, 2]
    slots = [9, 2, -1, 23, 0, 14, 7]
    rot = {"dims": rotary, "base": 10000.0, "scaling": {"factor": 6.0, "low": 1.0, "high": 3.0, "original": 64}}
    frequencies = plain.rotary_frequencies(rot) if rotary else []
    inv_freq = dev(torch.tensor(frequencies, dtype=torch.float64).float()) if rotary else None
    q_out = torch.zeros(tokens, H * 2 * d, dtype=dtype, device="cuda")
    k_pages = torch.zeros(pages, G, page, 2 * d, dtype=dtype, device="cuda")
    v_pages = torch.zeros(pages, G, page, dv, dtype=dtype, device="cuda")
    differential.bias_rope_cache(dev(qkv), dev(bias), i32(positions), i32(slots), inv_freq, rotary, q_out, k_pages,
                                 v_pages, H, G, d, dv, page)
    single = [float(f) for f in torch.tensor(frequencies, dtype=torch.float64).float().double()]   # as the kernel holds them
    tolerance = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    for t in range(tokens):
        row = qkv[t].double() + bias.double()
        # The angle is a float32 product: at a far position the plain rule is followed with frequencies that
        # give, at this position, the angle as float32 rounds it.
        position = positions[t]
        as_rounded = [float(torch.tensor(position * f, dtype=torch.float32)) / position if position else f for f in single]
        units = row[:(H + G) * 2 * d].view(-1, d)
        turned = torch.stack([plain.rotate(unit, position, as_rounded) for unit in units]) if rotary else units
        assert torch.allclose(q_out[t].cpu().double().view(-1, d), turned[:H * 2], **tolerance), t
        if slots[t] < 0:
            continue
        p, o = divmod(slots[t], page)
        assert torch.allclose(k_pages[p, :, o].cpu().double().reshape(-1, d), turned[H * 2:], **tolerance), t
        assert torch.allclose(v_pages[p, :, o].cpu().double(), row[(H + G) * 2 * d:].view(G, dv), **tolerance), t
    stored = {divmod(s, page) for s in slots if s >= 0}
    for p in range(pages):
        for o in range(page):
            if (p, o) not in stored:
                assert not k_pages[p, :, o].any() and not v_pages[p, :, o].any()


def plain_two_maps(q, keys, values, position, mask, scale, cap, lam, diff, eps):
    """One head: ``q`` ``[2, d]``, ``keys`` ``[n, 2, d]``, ``values`` ``[n, dv]`` of the positions 0 .. n - 1."""
    seen = [j for j in range(position + 1) if plain.sees(position, j, mask)]
    maps = []
    for m in range(2):
        score = (keys[seen, m] @ q[m]) * scale
        if cap:
            score = cap * torch.tanh(score / cap)
        maps.append(torch.softmax(score, dim=0) @ values[seen])
    return plain.rms(maps[0] - lam * maps[1], eps) * (1.0 - diff)


def paged(rows, page_size, pages_order, heads, size, dtype):
    """Scatter rows ``[n, heads, size]`` into pages taken in ``pages_order``."""
    n = rows.shape[0]
    store = torch.zeros(max(pages_order) + 1, heads, page_size, size, dtype=dtype)
    for j in range(n):
        store[pages_order[j // page_size], :, j % page_size] = rows[j].to(dtype)
    return store


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(5, 1, 48, 80, 90, 6), (6, 3, 10, 6, 7, 9), (2, 2, 64, 128, 100, 1), (8, 2, 64, 64, 64, 0),
                                   (3, 1, 32, 64, 1, 5), (2, 1, 128, 128, 300, 17), (4, 4, 16, 24, None, 0),
                                   (16, 1, 64, 128, 130, 3)])
def test_two_maps_at_the_edges_of_window_and_first_positions(dtype, shape):
    """A request that decodes one token over 700 keys, one whose last 35 tokens over scattered pages are this
    step's portion, one that starts.  In each map of a head one query is scaled so that it points at one key:
    the oldest inside the window, the one just outside it, the last of the kept first positions, the first
    behind them, keys on both sides of a page border and a key hundreds of positions back; the two maps point
    at different keys, so a swap of the maps, a lost lambda or a window that is one off moves the output."""
    from vllm_from_scratch_b200.kernels import differential
    H, G, d, dv, window, keep = shape
    g = torch.Generator().manual_seed(17)
    page, eps, scale, cap, lam, diff = 16, 1e-5, 10.0 / d, 30.0, 0.37, 0.6
    mask = None if window is None else {"size": window, "keep_first": keep}
    lengths, fresh = [700, 333, 5], [1, 35, 5]
    sequences = []
    for n in lengths:
        q = torch.randn(n, H, 2, d, generator=g)
        k = torch.randn(n, G, 2, d, generator=g)
        v = torch.randn(n, G, dv, generator=g)
        sequences.append([q, k, v])
    # Queries that point: query i of head h, map m, is a multiple of the key at the position it points to.
    reach = window if window is not None else 650
    for (q, k, v), n, new in zip(sequences, lengths, fresh):
        for row, i in enumerate(range(n - new, n)):
            targets = [i - reach + 1, i - reach, keep - 1, keep, (i // page) * page - 1, (i // page) * page, i - 640, i]
            for h in range(H):
                for m in range(2):
                    j = targets[(row + h + 3 * m) % len(targets)]
                    if 0 <= j <= i:
                        key = k[j, h // (H // G), m]
                        q[i, h, m] = key * (d / float(key @ key))       # scores 10 at its key
    sequences = [[rounded(t, dtype) for t in s] for s in sequences]
    order = torch.randperm(sum(-(-n // page) for n in lengths), generator=g).tolist()
    tables, at = [], 0
    for n in lengths:
        count = -(-n // page)
        tables.append(order[at:at + count])
        at += count
    k_pages = torch.zeros(len(order), G, page, 2 * d, dtype=dtype)
    v_pages = torch.zeros(len(order), G, page, dv, dtype=dtype)
    for (q, k, v), table, n in zip(sequences, tables, lengths):
        for j in range(n):
            k_pages[table[j // page], :, j % page] = k[j].reshape(G, 2 * d).to(dtype)
            v_pages[table[j // page], :, j % page] = v[j].to(dtype)
    width = max(len(t) for t in tables)
    block_table = i32([t + [-1] * (width - len(t)) for t in tables])
    q_rows = torch.cat([s[0][n - new:].reshape(new, H * 2 * d) for s, n, new in zip(sequences, lengths, fresh)])
    starts = [0]
    for new in fresh:
        starts.append(starts[-1] + new)
    out = torch.empty(sum(fresh), H * dv, dtype=dtype, device="cuda")
    differential.diff_paged_attention(dev(q_rows, dtype), dev(k_pages), dev(v_pages), out, i32(starts), i32(lengths),
                                      block_table, H, G, d, dv, page, scale, cap, window, keep, lam, eps, 1.0 - diff,
                                      max_query_len=max(fresh), max_seq_len=max(lengths), num_decode=1)
    got = out.cpu().double().view(sum(fresh), H, dv)
    row = 0
    worst = 0.0
    for (q, k, v), n, new in zip(sequences, lengths, fresh):
        for i in range(n - new, n):
            for h in range(H):
                kv = h // (H // G)
                want = plain_two_maps(q[i, h], k[:, kv], v[:, kv], i, mask, scale, cap, lam, diff, eps)
                worst = max(worst, float((got[row, h] - want).abs().max()))
            row += 1
    # the outputs are of unit root mean square times 0.4
    assert worst <= (2e-5 if dtype == torch.float32 else 2e-2), worst


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_maps_without_a_cap_and_with_pages_given_back(dtype):
    """No cap on the scores; the pages between the kept first positions and the window have been given back
    (their entries are negative) and must not be read."""
    from vllm_from_scratch_b200.kernels import differential
    H, G, d, dv, window, keep, page = 2, 1, 32, 32, 40, 10, 8
    g = torch.Generator().manual_seed(5)
    n, new = 200, 3
    q = rounded(torch.randn(n, H, 2, d, generator=g), dtype)
    k = rounded(torch.randn(n, G, 2, d, generator=g), dtype)
    v = rounded(torch.randn(n, G, dv, generator=g), dtype)
    count = -(-n // page)
    table = list(range(count))
    first_needed = (n - new - window + 1) // page
    for index in range(-(-keep // page), first_needed):
        table[index] = -1
    k_pages = paged(k.reshape(n, G, 2 * d), page, list(range(count)), G, 2 * d, dtype)
    v_pages = paged(v, page, list(range(count)), G, dv, dtype)
    for index, entry in enumerate(table):
        if entry < 0:           # what lies in a page that was given back is someone else's by now
            k_pages[index] = 1.0e4
            v_pages[index] = 1.0e4
    out = torch.empty(new, H * dv, dtype=dtype, device="cuda")
    differential.diff_paged_attention(dev(q[n - new:].reshape(new, -1), dtype), dev(k_pages), dev(v_pages), out,
                                      i32([0, new]), i32([n]), i32([table]), H, G, d, dv, page, 0.2, None, window, keep,
                                      -0.8, 1e-6, 0.25)
    got = out.cpu().double().view(new, H, dv)
    mask = {"size": window, "keep_first": keep}
    for row, i in enumerate(range(n - new, n)):
        for h in range(H):
            want = plain_two_maps(q[i, h], k[:, 0], v[:, 0], i, mask, 0.2, None, -0.8, 0.75, 1e-6)
            assert float((got[row, h] - want).abs().max()) <= (2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(16, 4, 2), (3, 3, 3), (2, 5, 3), (8, 0, 4), (1, 1, 2), (12, 4, 1)])
def test_softmax_routing_with_identity_experts(dtype, sizes):
    """Chosen experts and weights against the plain rule: a softmax over all router outputs, the choice on
    score + correction, the weights the chosen scores over their sum.  The corrections are large enough to
    make the choice differ from the choice by plain scores."""
    from vllm_from_scratch_b200.kernels import grouped
    experts, identity, top = sizes
    outputs, hidden, tokens = experts + identity, 40, 33
    g = torch.Generator().manual_seed(outputs * 10 + top)
    x = torch.randn(tokens, hidden, generator=g).to(dtype)
    router = (torch.randn(outputs, hidden, generator=g) * 0.4).to(torch.bfloat16).float()
    correction = (torch.randn(outputs, generator=g) * 0.3).to(torch.bfloat16).float()
    ids = torch.empty(tokens, top, dtype=torch.int32, device="cuda")
    weights = torch.empty(tokens, top, dtype=torch.float32, device="cuda")
    grouped.route_experts(dev(x), dev(router), dev(correction), ids, weights, top, scoring="softmax", renormalise=True)
    w = {"router": router, "correction": correction}
    plain_by_scores = 0
    for t in range(tokens):
        chosen, picked = plain.route(w, {"top": top}, x[t].double())
        scores = torch.softmax(router.double() @ x[t].double(), dim=0)
        margin = torch.topk(scores + correction.double(), min(top + 1, outputs)).values
        if outputs > top and float(margin[-2] - margin[-1]) < 1e-4:
            continue                                        # a close call: either choice is right
        assert ids[t].tolist() == chosen, t
        assert torch.allclose(weights[t].cpu().double(), torch.stack(picked), rtol=1e-5, atol=1e-7)
        plain_by_scores += set(chosen) != set(torch.topk(scores, top).indices.tolist())
    assert outputs == top or plain_by_scores > 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(64, 40, 6, 2, 2, 24), (50, 33, 2, 5, 3, None), (128, 96, 16, 4, 2, 128), (37, 9, 3, 0, 3, 7),
                                   (96, 24, 1, 3, 4, 16)])
@pytest.mark.parametrize("tokens", [70, 5])
def test_experts_identity_experts_and_a_shared_expert(dtype, sizes, tokens):
    """The whole routed feed-forward as a part, from tensors under the checkpoint's names: lists per expert
    without the identity experts' pairs, the grouped products, the weighted sum in which an identity expert
    adds the token's own input, and the expert that every token passes."""
    from vllm_from_scratch_b200.parts.base import FEED_FORWARDS, PartEnv, StepContext
    hidden, inter, experts, identity, top, shared = sizes
    g = torch.Generator().manual_seed(hidden + tokens)
    params = {"num_experts": experts, "identity_experts": identity, "top": top, "intermediate_size": inter,
              "scoring": "softmax", "renormalise": True, "correction": True, "shared_intermediate_size": shared}
    part = FEED_FORWARDS.get("routed_experts")(params, PartEnv(hidden, dtype, torch.device("cuda"), "mlp."))
    w = {}
    for name, info in part.expected_weights().items():
        w[name] = (torch.randn(info.shape, generator=g) * (0.5 if name == "correction" else info.shape[-1] ** -0.5)
                   ).to(torch.bfloat16)
    part.load_weights({name: dev(t, torch.float32 if part.expected_weights()[name].kind == "vector" else dtype)
                       for name, t in w.items()})
    x = torch.randn(tokens, hidden, generator=g).to(dtype)
    got = part.forward(dev(x), None).cpu().double()
    wd = {name: t.double() for name, t in w.items()}
    mlp = {"router": {"experts": experts, "identity": identity, "top": top}, "shared": {"ff": shared} if shared else None}
    want = torch.stack([plain.experts_feed_forward(wd, mlp, x[t].double()) for t in range(tokens)])
    bound = (2e-5 if dtype == torch.float32 else 3e-2) * float(want.abs().max())
    close = ((got - want).abs().max(dim=1).values <= bound)
    # bfloat16: a token whose choice hangs on a close call may take another expert
    assert int((~close).sum()) <= (0 if dtype == torch.float32 else tokens // 20), (~close).nonzero().flatten().tolist()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_gate(dtype):
    from vllm_from_scratch_b200.kernels import grouped
    g = torch.Generator().manual_seed(3)
    for tokens, inter in ((9, 77), (64, 320), (3, 8)):
        gate_up = (torch.randn(tokens, 2 * inter, generator=g) * 3).to(dtype)
        out = torch.empty(tokens, inter, dtype=dtype, device="cuda")
        grouped.gelu_mul(dev(gate_up), out)
        want = plain.gelu_tanh(gate_up[:, :inter].double()) * gate_up[:, inter:].double()
        assert torch.allclose(out.cpu().double(), want, **(dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32
                                                           else dict(rtol=1e-2, atol=1e-2)))


@pytest.mark.parametrize("shape", [(5, 1, 48, 80, 90, 6, 16), (8, 2, 32, 64, None, 0, 16), (4, 2, 64, 128, 600, 3, 32),
                                   (32, 1, 16, 16, 50, 2, 8), (2, 2, 80, 48, 1, 0, 16), (6, 2, 64, 128, 300, 300, 64),
                                   (12, 1, 32, 48, 200, 5, 16), (32, 2, 16, 32, None, 0, 16), (8, 1, 64, 64, 700, 1, 16)])
def test_tensor_core_kernels_against_the_float32_arithmetic(shape):
    """bfloat16 batches of decoding requests (lengths 1, the window's and the kept positions' edges, some with
    their keys split over several blocks) ahead of portions of prompts (2, 63, 64, 65 and 200 tokens, with and
    without a past): the tensor-core kernels against the float32 kernel on the same pages."""
    from vllm_from_scratch_b200.kernels import differential
    H, G, d, dv, window, keep, page = shape
    g = torch.Generator().manual_seed(3)
    edge = window if window is not None else 400
    decoding = [1, 2, keep + 1, keep + 2, edge, edge + 1, edge + keep, edge + keep + 1, 900, 1500]
    decoding = [n for n in decoding if n >= 1]
    portions = [(2, 0), (63, 0), (64, 130), (65, 7), (200, edge + 3)]
    lengths = decoding + [new + past for new, past in portions]
    fresh = [1] * len(decoding) + [new for new, _ in portions]
    pages_of = [-(-n // page) for n in lengths]
    order = torch.randperm(sum(pages_of), generator=g).tolist()
    tables, at = [], 0
    for count in pages_of:
        tables.append(order[at:at + count])
        at += count
    width = max(pages_of)
    block_table = i32([t + [-1] * (width - len(t)) for t in tables])
    k_pages = dev(torch.randn(len(order), G, page, 2 * d, generator=g), torch.bfloat16)
    v_pages = dev(torch.randn(len(order), G, page, dv, generator=g), torch.bfloat16)
    q = dev(torch.randn(sum(fresh), H * 2 * d, generator=g) * 2.0, torch.bfloat16)
    starts = [0]
    for new in fresh:
        starts.append(starts[-1] + new)
    outs = []
    for tensor_cores, decode in ((False, 0), (True, len(decoding)), (True, 0)):
        out = torch.zeros(sum(fresh), H * dv, dtype=torch.bfloat16, device="cuda")
        differential.USE_TENSOR_CORES = tensor_cores
        try:
            differential.diff_paged_attention(q, k_pages, v_pages, out, i32(starts), i32(lengths), block_table, H, G, d,
                                              dv, page, d ** -0.5, 20.0, window, keep, 0.45, 1e-6, 0.4,
                                              max_query_len=max(fresh), max_seq_len=max(lengths), num_decode=decode)
        finally:
            differential.USE_TENSOR_CORES = True
        outs.append(out.float().cpu())
    assert differential.tensor_core_sizes_ok(d, dv)
    for got in outs[1:]:
        # outputs of root mean square 0.4, rounded to bfloat16: one step of the last place is 2 ** -8 at most
        assert float((got - outs[0]).abs().max()) <= 2 ** -7, float((got - outs[0]).abs().max())


def test_decode_splits_fill_the_gpu():
    from vllm_from_scratch_b200.kernels.differential import decode_splits, tensor_core_sizes_ok
    assert decode_splits(1, 1, 100, 148) == 1
    assert decode_splits(1, 1, 5000, 148) == 16
    assert decode_splits(8, 8, 1028, 148) == 4
    assert decode_splits(64, 8, 4096, 148) == 1          # pairs that fill the GPU by themselves are not split
    assert tensor_core_sizes_ok(48, 80) and tensor_core_sizes_ok(128, 256)
    assert not tensor_core_sizes_ok(10, 6) and not tensor_core_sizes_ok(64, 512) and not tensor_core_sizes_ok(512, 64)
