"""The Mupuvik design in the engine against the plain implementation: every kernel alone, whole models under every
way of cutting requests into steps, pages and slots that are used again, and greedy generation through the engine's
own entry point.  float32 runs are compared tightly, bfloat16 runs as a fraction of the largest logit."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers
import mupuvik_configs
import plain_mupuvik as plain

pytestmark = pytest.mark.gpu

CONFIGS, LENGTHS = mupuvik_configs.CONFIGS, mupuvik_configs.LENGTHS
# Bounds as a fraction of the sequence's largest logit, a few times the worst difference seen over all cuts.
F32_REL, BF16_REL = 2e-5, 0.06


def steady_choice(weights, raw):
    """The last coordinate of the stream is made a constant (the same number in every row of the token table, zero
    in the pairs' table and in the row of every matrix that writes into the stream), and every router reads it with
    factors 1.5 apart from expert to expert, in a shuffled order of its own in every layer, and the rest of it
    with a tenth of its random weights: the random part of a router's logits cannot bridge that, so the choice of
    experts never hangs on a close call between two scores, while the weights of the chosen still differ from token
    to token."""
    generator = torch.Generator().manual_seed(99)
    last = raw["width"] - 1
    weights["embed"][:, last] = 4.0 / raw["embedding"]["scale"]
    weights["bigram"][:, last] = 0.0
    for name, tensor in weights.items():
        if name.endswith((".o", ".down")):
            tensor[last, :] = 0.0
        if name.endswith(".router"):
            levels = 1.5 * torch.randperm(tensor.shape[0], generator=generator).float()
            tensor.mul_(0.1)
            tensor[:, last] = (levels - levels.mean()).to(tensor.dtype)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """Stored in bfloat16: both run modes and the plain implementation then read the same numbers.  The float32
    runs route as the random weights say.  The bfloat16 runs get models whose choice of experts is steady
    (``steady_choice``): the rounding of the stream moves a router's scores by about a hundredth, which in a
    random model turns a close call the other way every few dozen tokens and changes that row, and through the
    caches and states the rows behind it, by far more than rounding."""
    made = {}
    for i, (name, (raw, _)) in enumerate(CONFIGS.items()):
        made[name, "float32"] = helpers.make_model_folder(tmp_path_factory.mktemp("mupuvik"), raw, seed=21 + i,
                                                          dtype=torch.bfloat16)
        made[name, "bfloat16"] = helpers.make_model_folder(tmp_path_factory.mktemp("mupuvik_steady"), raw, seed=21 + i,
                                                           dtype=torch.bfloat16, special=steady_choice)
    return made


def load_plain(folder, raw):
    from safetensors import safe_open
    weights = {}
    with safe_open(str(folder / "model.safetensors"), "pt") as handle:
        for key in handle.keys():
            weights[key] = handle.get_tensor(key)
    return plain.PlainMupuvik(raw, weights, torch.float64)


@pytest.fixture(scope="module")
def references(folders):
    out = {}
    for (name, dtype), folder in folders.items():
        raw = CONFIGS[name][0]
        model = load_plain(folder, raw)
        sequences = {rid: helpers.random_tokens(raw["vocab"], n, seed=sum(map(ord, name + rid)))
                     for rid, n in LENGTHS[name].items()}
        out[name, dtype] = (sequences, {rid: model.feed(model.new_state(), tokens).float() for rid, tokens in sequences.items()})
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
    "tail": lambda lengths: helpers.cut_tail_one_by_one(lengths, 45),
    "portions": lambda lengths: helpers.cut_changing_portions(lengths, seed=1),
    "one_by_one": lambda lengths: [[(rid, 1)] for rid, n in lengths.items() if n <= 70 for _ in range(n)],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_each_request_alone(folders, references, name, cut, dtype):
    """Whole prompts, prompts whose last 45 tokens are decoded one by one (past every window of the small models),
    portions of changing sizes down to two tokens, and whole sequences decoded token by token: the same rows."""
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
    """Up to three live requests in three slots, portions beside single tokens, requests left out of steps, and a
    pool so small that the pages and the slot of a finished request (its recurrent states, its convolution inputs,
    its previous token) are handed out again at once."""
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name, dtype]
    steps = helpers.cut_mixed(LENGTHS[name], seed=seed, live=3)
    pages = sum(sorted((-(-n // page_size) for n in LENGTHS[name].values()), reverse=True)[:3])
    runner = make_runner(folders[name, dtype], dtype, page_size, pages, max_requests=3)
    results = helpers.run_schedule(runner, sequences, steps)
    compare(results, expected, dtype, f"{name}/mixed{seed}/{dtype}")
    assert runner.manager.stats()["requests"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_beside_single_tokens(folders, references, dtype):
    """Portions of 64 tokens and more beside decoded tokens: the portions' attention kernel at a row offset."""
    name = "C"
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name, dtype]
    steps = helpers.cut_mixed(LENGTHS[name], seed=7, live=3, sizes=(2, 33, 64, 100))
    pages = sum(sorted((-(-n // page_size) for n in LENGTHS[name].values()), reverse=True)[:3])
    runner = make_runner(folders[name, dtype], dtype, page_size, pages, max_requests=3)
    compare(helpers.run_schedule(runner, sequences, steps), expected, dtype, f"{name}/long portions/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_long_portions_run_in_segments(folders, references, name, dtype, monkeypatch):
    """Portions of 32 tokens and more are cut into segments of about 16 that run side by side, each from an empty
    state, and are then corrected by the state they should have started from (decays per head in the scan, per
    head and key channel in the gated linear attention): the same rows, for whole prompts, for portions that
    start in the middle of a sequence, and beside single tokens."""
    from vllm_from_scratch_b200.kernels import mixing
    monkeypatch.setattr(mixing, "SCAN_SEGMENT", 16)
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name, dtype]
    for label, steps in (("whole", helpers.cut_whole(LENGTHS[name])),
                         ("mixed", helpers.cut_mixed(LENGTHS[name], seed=5, live=3, sizes=(2, 33, 40, 64, 100)))):
        pages = sum(sorted((-(-n // page_size) for n in LENGTHS[name].values()), reverse=True)[:3])
        runner = make_runner(folders[name, dtype], dtype, page_size, pages, max_requests=3)
        results = helpers.run_schedule(runner, sequences, steps)
        compare(results, expected, dtype, f"{name}/segments/{label}/{dtype}")


def test_long_decoding_keeps_the_state(folders, references):
    """A short prompt and 140 tokens decoded one by one through recurrences, the convolution and windows that
    have long passed the prompt."""
    raw, page_size = CONFIGS["A"]
    sequences, expected = references["A", "float32"]
    runner = make_runner(folders["A", "float32"], "float32", page_size, 12)
    steps = [[("g", 10)]] + [[("g", 1)] for _ in range(140)]
    results = helpers.run_schedule(runner, {"g": sequences["g"]}, steps)
    compare(results, expected, "float32", "A/long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(folders, dtype):
    """``LLM.generate`` (scheduler, token budget, graph replay of decode steps, steps queued ahead) gives the tokens
    that the plain implementation's argmax gives, for prompts of unequal lengths that are cut by the token budget
    and run side by side."""
    import vllm_from_scratch_b200 as engine
    raw, page_size = CONFIGS["A"]
    model = load_plain(folders["A", dtype], raw)
    prompts = [helpers.random_tokens(raw["vocab"], n, seed=40 + n) for n in (5, 37, 1, 60)]
    new_tokens = 12
    llm = engine.LLM(str(folders["A", dtype]), dtype=dtype, max_model_len=128, block_size=page_size, num_gpu_blocks=40,
                     max_num_seqs=3, max_num_batched_tokens=24)
    outputs = llm.generate(prompts, engine.SamplingParams(max_tokens=new_tokens, temperature=0.0, ignore_eos=True))
    assert llm.engine.decode_graphs is not None and llm.engine.decode_graphs.replays > 0
    for prompt, output in zip(prompts, outputs):
        state = model.new_state()
        logits = model.feed(state, prompt)
        for index, token in enumerate(output.token_ids):
            row = logits[-1]
            best = int(row.argmax())
            if token != best:
                # bfloat16 may swap two tokens that the plain implementation puts within its noise
                gap = float(row[best] - row[token]) / float(row.abs().max())
                assert dtype == "bfloat16" and gap < 0.03, (index, token, best, gap)
            logits = model.feed(state, [token])
        assert len(output.token_ids) == new_tokens
    llm.engine.shutdown()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folders, references, tmp_path, dtype):
    """``bin/trace_run`` in a process of its own: a mixed schedule of up to four live requests over a pool of 4 x 128
    positions and four state slots."""
    name = "A"
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name, dtype]
    lengths = {rid: min(n, 128) for rid, n in LENGTHS[name].items()}
    sequences = {rid: toks[:lengths[rid]] for rid, toks in sequences.items()}
    steps = helpers.cut_mixed(lengths, seed=5, live=4)
    lines = helpers.schedule_to_trace(sequences, steps)
    out = tmp_path / "out"
    root = Path(__file__).resolve().parent.parent
    process = subprocess.run(
        [sys.executable, str(root / "bin" / "trace_run"), "--model", str(folders[name, dtype]), "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(4 * 128)],
        input="\n".join(json.dumps(line) for line in lines) + "\n", capture_output=True, text=True,
        timeout=900, env={**os.environ, "PYTHONPATH": ""})
    assert process.returncode == 0, process.stderr[-3000:]
    assert [l for l in process.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(lines))]
    done = {rid: 0 for rid in sequences}
    bound_rel = F32_REL if dtype == "float32" else BF16_REL
    for line in lines:
        data = np.fromfile(out / f"{line['step']}.f32", dtype="<f4").reshape(-1, raw["vocab"])
        at = 0
        for entry in line["entries"]:
            n = len(entry["tokens"])
            reference = expected[entry["id"]][done[entry["id"]]:done[entry["id"]] + n]
            diff = (torch.from_numpy(data[at:at + n].copy()) - reference).abs().max()
            assert float(diff) <= bound_rel * float(expected[entry["id"]].abs().max()), (line["step"], entry["id"], float(diff))
            at += n
            done[entry["id"]] += n
        assert at == data.shape[0]


# ------------------------------------------------------------------- kernels alone
def dev(tensor, dtype=None):
    return tensor.to("cuda", dtype) if dtype is not None else tensor.to("cuda")


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels(dtype):
    from vllm_from_scratch_b200 import kernels
    g = torch.Generator().manual_seed(3)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    tokens, heads, dv = 7, 5, 12
    x = torch.randn(tokens, heads * dv, generator=g).to(dtype)
    proj = torch.randn(tokens, 31 + heads, generator=g).to(dtype)          # the gates are the row's last columns
    out = torch.empty(tokens, heads * dv, dtype=dtype, device="cuda")
    kernels.head_gate(dev(x), dev(proj), 31, out, heads, 0.75)
    want = (x.double().view(tokens, heads, dv) * torch.sigmoid(proj[:, 31:].double())[:, :, None]).reshape(tokens, -1) * 0.75
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
    x_d = dev(x)
    kernels.head_gate(x_d, dev(proj), 31, x_d, heads)                       # in place
    assert torch.allclose(x_d.cpu().double(), want / 0.75, atol=tol, rtol=tol)
    a, b = torch.randn(9, 33, generator=g).to(dtype), torch.randn(9, 33, generator=g).to(dtype)
    out = torch.empty(9, 33, dtype=dtype, device="cuda")
    kernels.scaled_sum(dev(a), 0.6, dev(b), -1.5, out)
    assert torch.allclose(out.cpu().double(), a.double() * 0.6 - b.double() * 1.5, atol=tol, rtol=tol)
    # a norm per head with one vector for all heads, the silu of the gate behind it
    width, groups, eps = 96, 4, 1e-5
    y = torch.randn(tokens, width, generator=g)
    gate = torch.randn(tokens, width + 40, generator=g).to(dtype)
    vector = torch.randn(width // groups, generator=g)
    out = torch.empty(tokens, width, dtype=dtype, device="cuda")
    kernels.gated_group_norm(dev(y), dev(gate), dev(vector.repeat(groups)), out, groups, False, eps, silu_behind=True)
    want = (plain.norm_plain(y.double().view(tokens, groups, -1), vector.double(), eps).reshape(tokens, width)
            * plain.silu(gate[:, :width].double()))
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)


def test_bigram_embedding_scales_the_token_row_alone():
    from vllm_from_scratch_b200 import kernels
    g = torch.Generator().manual_seed(4)
    vocab, hidden, buckets, mul_prev, mul_cur, scale = 50, 24, 7, 3, 10, 0.25
    table, bigram = torch.randn(vocab, hidden, generator=g), torch.randn(buckets + 1, hidden, generator=g)
    previous = torch.zeros(3, 1, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    cfg = {"embedding": {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}}
    weights = {"embed": table, "bigram": bigram}
    tokens = [4, 49, 0, 17]
    out = torch.empty(3, hidden, device="cuda")
    kernels.bigram_embedding(dev(table), dev(bigram), i32(tokens[:3]), i32([0, 1, 2]), i32([0, 0, 0]), i32([0, 3]),
                             i32([1]), previous, out, mul_prev, mul_cur, flag, scale=scale)
    want = torch.stack([plain.embed_row(weights, cfg, before, token)
                        for before, token in zip([None] + tokens[:2], tokens[:3])])
    assert torch.allclose(out.cpu(), want, atol=1e-6)
    out = torch.empty(1, hidden, device="cuda")
    kernels.bigram_embedding(dev(table), dev(bigram), i32(tokens[3:]), i32([3]), i32([0]), i32([0, 1]), i32([1]),
                             previous, out, mul_prev, mul_cur, flag, scale=scale)
    assert torch.allclose(out.cpu()[0], plain.embed_row(weights, cfg, tokens[2], tokens[3]), atol=1e-6)
    assert flag.item() == 0 and previous[1, 0].item() == tokens[3]


FORMS = {
    # norm over the whole projection, biases, a window, an ordinary softmax
    "windowed": dict(norm="whole", bias=True, rot=None, window=40, sink=False),
    # norm per head, neighbours rotated over part of the head, every earlier key, one more in the denominator
    "rotary_sink": dict(norm="head", bias=False, rot=(10000.0, None), window=None, sink=True),
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(6, 2, 20, 36), (4, 2, 64, 64), (8, 1, 128, 128), (3, 3, 24, 8)])
@pytest.mark.parametrize("form", list(FORMS))
def test_attention_forms_far_keys_window_edges_and_page_borders(dtype, shape, form):
    """Two requests that decode one token (one over 1500 keys) ahead of a request of 333 positions in scattered pages
    whose last 40 tokens are this step's portion and of one that starts.  Queries are made to point at chosen keys
    (a far one at position 3, the keys just inside and just outside the window, the keys on both sides of page
    borders, the newest), so that a kernel that lost one of them, or saw one too many, would give another row.  One
    head's queries point away from every key, so that the one in the denominator takes most of its weight.  Keys
    and values of one size of 64 or 128 run on the tensor-core kernels in bfloat16, everything else in the
    float32-arithmetic kernel."""
    from vllm_from_scratch_b200 import kernels
    spec = FORMS[form]
    g = torch.Generator().manual_seed(5)
    H, G, d, dv = shape
    page, eps, scale = 16, 1e-5, 16.0 / d
    window, sink = spec["window"], spec["sink"]
    rot_dims = 0
    inv_freq = None
    if spec["rot"] is not None:
        rot_dims = d // 2
        base = spec["rot"][0]
        inv_freq = torch.tensor([base ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)], dtype=torch.float64)
    lengths, fresh = [1500, 200, 333, 3], [1, 1, 40, 3]
    whole = spec["norm"] == "whole"
    qw = torch.rand(H * d if whole else d, generator=g) + 0.5
    kw = torch.rand(G * d if whole else d, generator=g) + 0.5
    bias = torch.randn((H + G) * d + G * dv, generator=g) * 0.1 if spec["bias"] else None
    sequences = []
    for n in lengths:
        q, k, v = torch.randn(n, H, d, generator=g), torch.randn(n, G, d, generator=g), torch.randn(n, G, dv, generator=g)
        sequences.append([q.to(dtype).double(), k.to(dtype).double(), v.to(dtype).double()])

    def prepared(rows, weight, offset, position):
        """Bias, norm and rotation of one token's heads ``[heads, d]`` as the mixer defines them."""
        heads = rows.shape[0]
        if bias is not None:
            rows = rows + bias[offset:offset + heads * d].double().view(heads, d)
        if whole:
            rows = plain.norm_plain(rows.reshape(-1), weight.double(), eps).view(heads, d)
        else:
            rows = plain.norm_plain(rows, weight.double(), eps)
        if inv_freq is not None:
            rows = plain.rotate_pairs(rows, position, spec["rot"][0], rot_dims)
        return rows

    def point(sequence, at, key, strength=4.0):
        # The query of every head becomes its key's direction, which survives the norms roughly; where part of the
        # head is rotated, only in the part that is not (the rest of the query is zero).
        q, k, _ = sequence
        for head in range(H):
            q[at, head] = (k[key, head // (H // G)] * strength).to(dtype).double()
            q[at, head, :rot_dims] = 0.0

    targets = {300: 3, 301: 15, 302: 16, 303: 17, 304: 255, 305: 256, 306: 304, 332: 0}
    if window is not None:
        targets.update({310: 310 - window + 1, 311: 311 - window, 312: 312 - window + 2})    # inside, outside, inside
    for at, key in targets.items():
        point(sequences[2], at, key)
    point(sequences[0], 1499, 3)
    point(sequences[1], 199, 199 - (window or 40) + 1)
    if sink:
        for sequence in sequences:
            sequence[0][:, 0] = -sequence[1][:, 0] * 3.0                    # head 0 points away from its own key
    tokens = sum(fresh)
    qkv = torch.zeros(tokens, (H + G) * d + G * dv + 5, dtype=torch.float64)        # five more columns at the row's end
    want = torch.zeros(tokens, H * dv, dtype=torch.float64)
    without_sink = torch.zeros_like(want)
    positions, slots, tables, starts, row = [], [], [], [0], 0
    pool_pages = 160
    pages_free = list(torch.randperm(pool_pages, generator=g).tolist())
    k_pool = torch.zeros(pool_pages, G, page, d, dtype=dtype)
    v_pool = torch.zeros(pool_pages, G, page, dv, dtype=dtype)
    for (q, k, v), n, new in zip(sequences, lengths, fresh):
        table = [pages_free.pop() for _ in range(-(-n // page))]
        tables.append(table)
        kn = torch.stack([prepared(k[position], kw, H * d, position) for position in range(n)])
        vb = v if bias is None else v + bias[(H + G) * d:].double().view(G, dv)
        for position in range(n - new):        # what earlier steps left in the pages
            k_pool[table[position // page], :, position % page] = kn[position].to(dtype)
            v_pool[table[position // page], :, position % page] = vb[position].to(dtype)
        kn_seen, vb_seen = kn.to(dtype).double(), vb.to(dtype).double()      # read back from the pages in the run dtype
        for position in range(n - new, n):
            qkv[row, :(H + G) * d + G * dv] = torch.cat([q[position].reshape(-1), k[position].reshape(-1), v[position].reshape(-1)])
            qn = prepared(q[position], qw, 0, position).to(dtype).double()
            first = 0 if window is None else max(0, position - window + 1)
            want[row] = plain.attend(qn, kn_seen[:position + 1], vb_seen[:position + 1], scale, H // G, first, sink).reshape(-1)
            without_sink[row] = plain.attend(qn, kn_seen[:position + 1], vb_seen[:position + 1], scale, H // G, first, False).reshape(-1)
            positions.append(position)
            slots.append(table[position // page] * page + position % page)
            row += 1
        starts.append(row)
    width = max(len(t) for t in tables)
    table_t = torch.full((len(lengths), width), -1, dtype=torch.int32)
    for r, table in enumerate(tables):
        table_t[r, :len(table)] = torch.tensor(table)
    k_d, v_d = dev(k_pool), dev(v_pool)
    q_out = torch.empty(tokens, H * d, dtype=dtype, device="cuda")
    kernels.qk_prepare_cache(dev(qkv, dtype), None if bias is None else dev(bias), i32(positions), i32(slots), dev(qw), dev(kw),
                             spec["norm"], eps, None if inv_freq is None else dev(inv_freq, torch.float32), rot_dims, True,
                             q_out, k_d, v_d, H, G, d, dv, page)
    # Rows a multiple of four numbers long take the kernel's form of four numbers a lane: the same queries and pages.
    wider = torch.zeros(tokens, (H + G) * d + G * dv + 8, dtype=torch.float64)
    wider[:, :qkv.shape[1]] = qkv
    k_d2, v_d2, q_out2 = dev(k_pool), dev(v_pool), torch.empty_like(q_out)
    kernels.qk_prepare_cache(dev(wider, dtype), None if bias is None else dev(bias), i32(positions), i32(slots), dev(qw), dev(kw),
                             spec["norm"], eps, None if inv_freq is None else dev(inv_freq, torch.float32), rot_dims, True,
                             q_out2, k_d2, v_d2, H, G, d, dv, page)
    close = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    for one, other in ((q_out, q_out2), (k_d, k_d2), (v_d, v_d2)):
        assert torch.allclose(one.float(), other.float(), **close)
    sinks = torch.zeros(H, device="cuda") if sink else None
    tol = 2e-5 if dtype == torch.float32 else 4e-2

    def check(out, what, rows=slice(None)):
        diff = (out.cpu().double() - want[rows]).abs().max(dim=1).values
        assert float(diff.max()) < tol * float(want.abs().max()), (what, diff)

    out = torch.empty(tokens, H * dv, dtype=dtype, device="cuda")
    kernels.biased_paged_attention(q_out, k_d, v_d, out, i32(starts), i32(lengths), dev(table_t), None, H, G, d, dv,
                                   page, scale, window, max(fresh), max(lengths), 2, sinks=sinks)
    check(out, "as the engine calls it")
    out = torch.empty(tokens, H * dv, dtype=dtype, device="cuda")
    kernels.biased_paged_attention(q_out, k_d, v_d, out, i32(starts), i32(lengths), dev(table_t), None, H, G, d, dv,
                                   page, scale, window, sinks=sinks)
    check(out, "float32 arithmetic")
    # A gate per token and head applied as the rows are written, into the first columns of wider rows.
    gates = torch.randn(tokens, 3 + H, generator=g).to(dtype)
    gated = (want.view(tokens, H, dv) * (0.7 * torch.sigmoid(gates[:, 3:].double()))[:, :, None]).reshape(tokens, -1)
    for cores in (True, False):
        wide = torch.zeros(tokens, H * dv + 8, dtype=dtype, device="cuda")
        kernels.biased_paged_attention(q_out, k_d, v_d, wide[:, :H * dv], i32(starts), i32(lengths), dev(table_t), None, H, G,
                                       d, dv, page, scale, window, max(fresh) if cores else None, max(lengths), 2,
                                       sinks=sinks, gate=dev(gates), gate_column=3, gate_factor=0.7)
        diff = (wide[:, :H * dv].cpu().double() - gated).abs().max()
        assert float(diff) < tol * float(want.abs().max()), ("gated", cores, float(diff))
        assert not wide[:, H * dv:].any()
    out = torch.empty(2, H * dv, dtype=dtype, device="cuda")                # the single tokens alone: a decode step
    kernels.biased_paged_attention(q_out[:2], k_d, v_d, out, i32(starts[:3]), i32(lengths[:2]), dev(table_t[:2]), None,
                                   H, G, d, dv, page, scale, window, 1, max(lengths), 0, sinks=sinks)
    check(out, "decode step", slice(0, 2))
    # The oracle itself shows what the test is after: a pointed query singles its key out where the key is visible
    # and not where the window has passed it, and the one in the denominator moves head 0 by much.
    if d >= 64:
        v2 = sequences[2][2] if bias is None else sequences[2][2] + bias[(H + G) * d:].double().view(G, dv)
        for at, key in targets.items():
            r = 2 + at - (lengths[2] - fresh[2])
            close = float((want[r, (H - 1) * dv:] - v2[key, G - 1]).abs().max()) < 0.35 * float(v2[key, G - 1].abs().max())
            visible = window is None or at - key < window
            assert close == visible, (at, key, visible)
    if sink:
        assert float((want[:, :dv] - without_sink[:, :dv]).abs().max()) > 0.3 * float(without_sink[:, :dv].abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("segments", [False, True])
@pytest.mark.parametrize("shape", [(3, 40, 72), (2, 8, 16), (1, 132, 20), (6, 48, 32)])
def test_gated_linear_attention_in_portions(dtype, shape, segments, monkeypatch):
    """Three requests advance through several steps in slots of their own, in portions of 1 to 21 tokens; the slot
    of the first is then used again by a new request.  The decays differ from channel to channel (logits from -4 to
    6, so that some rows of the state are nearly kept and others nearly forgotten at every token).  ``segments``:
    portions of 8 tokens and more run as segments of about 4 side by side."""
    from vllm_from_scratch_b200 import kernels
    from vllm_from_scratch_b200.kernels import mixing
    if segments:
        monkeypatch.setattr(mixing, "SCAN_SEGMENT", 4)
    H, n, dv = shape
    g = torch.Generator().manual_seed(6)
    tau = 3.0
    stride = 5 + H * (2 * n + dv)
    offsets = (5 + H * dv, 5 + H * dv + H * n, 5)         # v first, then q, then k, behind five other columns
    gate_bias = torch.linspace(-4.0, 6.0, H * n)
    state = torch.zeros(5, H, n, dv, device="cuda")
    plans = {0: [1, 1, 21, 2, 1], 3: [17, 1, 1, 1, 1], 1: [2, 3, 1, 16, 5]}
    projections = {slot: torch.randn(sum(sizes), stride, generator=g).to(dtype) for slot, sizes in plans.items()}
    logits = {slot: torch.randn(sum(sizes), 3 + H * n, generator=g).to(dtype) for slot, sizes in plans.items()}

    def oracle(proj, z):
        S = [torch.zeros(n, dv, dtype=torch.float64) for _ in range(H)]
        rows = []
        for row, z_row in zip(proj.double(), z.double()):
            q = row[offsets[0]:offsets[0] + H * n].view(H, n) * n ** -0.5
            k = row[offsets[1]:offsets[1] + H * n].view(H, n)
            alpha = torch.sigmoid(z_row[3:] + gate_bias.double()).pow(1.0 / tau).view(H, n)
            rows.append(plain.gated_linear_attention_step(q, k, row[5:5 + H * dv].view(H, dv), alpha, S).reshape(-1))
        return torch.stack(rows)

    want = {slot: oracle(projections[slot], logits[slot]) for slot in plans}
    done = {slot: 0 for slot in plans}
    got = {slot: [] for slot in plans}
    tol = 1e-4 if dtype == torch.float32 else 2e-2

    def run(pieces, z_pieces, starts, order, y):
        longest = max(b - a for a, b in zip(starts, starts[1:])) if segments else None
        kernels.gated_linear_attention(dev(torch.cat(pieces)), offsets, dev(torch.cat(z_pieces)), 3, dev(gate_bias), tau,
                                       n ** -0.5, i32(starts), i32(order), state, y, H, n, dv, longest)

    for step in range(5):
        order = [3, 0, 1] if step % 2 else [1, 3, 0]
        pieces, z_pieces, starts = [], [], [0]
        for slot in order:
            size = plans[slot][step]
            pieces.append(projections[slot][done[slot]:done[slot] + size])
            z_pieces.append(logits[slot][done[slot]:done[slot] + size])
            starts.append(starts[-1] + size)
        y = torch.empty(starts[-1], H * dv, device="cuda")
        run(pieces, z_pieces, starts, order, y)
        for index, slot in enumerate(order):
            got[slot].append(y[starts[index]:starts[index + 1]].cpu())
            done[slot] += plans[slot][step]
    for slot in plans:
        result = torch.cat(got[slot]).double()
        assert float((result - want[slot]).abs().max()) < tol * float(want[slot].abs().max()), slot
    state[0].zero_()                                    # what the cache does when it hands the slot out again
    y = torch.empty(4, H * dv, device="cuda")
    run([projections[3][:4]], [logits[3][:4]], [0, 4], [0], y)
    assert float((y.cpu().double() - want[3][:4]).abs().max()) < tol * float(want[3].abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens", [5, 90, 300])
@pytest.mark.parametrize("top", [1, 3])
def test_experts_weighted_on_their_input(dtype, tokens, top):
    """The routed feed-forward as a part against the plain one, for steps of few rows, of a few tiles and of so many
    rows that the bfloat16 run takes the library's grouped product; limits that cut many of the gates."""
    from vllm_from_scratch_b200.parts import FEED_FORWARDS, PartEnv
    from vllm_from_scratch_b200.parts.base import StepContext
    g = torch.Generator().manual_seed(8 + tokens + top)
    hidden, experts, ff, shared_ff = 64, 5, 32, 48
    cfg = {"expert": {"ff": ff, "limit": 0.4}, "router": {"experts": experts, "top": top}, "shared": {"ff": shared_ff, "limit": 0.7}}
    weights = {"router": torch.randn(experts, hidden, generator=g) * 0.3}
    for name, width in [(f"e{e}.", ff) for e in range(experts)] + [("shared.", shared_ff)]:
        weights[name + "gate"] = (torch.randn(width, hidden, generator=g) * 0.2).to(dtype)
        weights[name + "up"] = (torch.randn(width, hidden, generator=g) * 0.2).to(dtype)
        weights[name + "down"] = (torch.randn(hidden, width, generator=g) * 0.2).to(dtype)
    x = torch.randn(tokens, hidden, generator=g).to(dtype)
    part = FEED_FORWARDS.get("routed_experts")(
        {"num_experts": experts, "top": top, "intermediate_size": ff, "correction": False, "weight_on_input": True,
         "activation": ("capped", 0.4, 1.702, 1.0), "shared_intermediate_size": shared_ff,
         "shared_activation": ("capped", 0.7, 1.702, 1.0)}, PartEnv(hidden, dtype, torch.device("cuda"), "mlp"))
    part.load_weights({name: dev(tensor, torch.float32 if name == "router" else dtype) for name, tensor in weights.items()})
    out = part.forward(dev(x), StepContext(tokens, 1, None, None, None, None, None, tokens, tokens)).cpu().double()
    plain_weights = {name: tensor.double() for name, tensor in weights.items()}
    want = torch.stack([plain.experts_step(plain_weights, cfg, row) for row in x.double()])
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert float((out - want).abs().max()) < tol * float(want.abs().max())
