"""The Tudulix design on the GPU against the plain NumPy restatement (``plain_tudulix.py``): each mechanism's kernels
alone, then whole models through the engine: prompts at once, decoding through the cache, portions of every size,
mixed batches with pages and slots that are freed and used again, window edges, long decoding, and greedy generation
through the Python entry point and the command line."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_tudulix as plain
from tiny_tudulix import CONFIGS, write_model

pytestmark = pytest.mark.gpu

FLOAT32_LIMIT = 2e-4   # of the logits' spread; 32-bit sums of a few hundred terms stay far below
BFLOAT16_LIMIT = 0.08


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("tudulix")
    return {name: write_model(root / name, config, 50 + seed) for seed, (name, config) in enumerate(CONFIGS.items())}


def tokens_for(config: dict, count: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, config["vocab"], size=count).tolist()


def load_engine(folder, dtype: str, max_tokens: int = 1024, **options):
    from lalamo_b200.engine.engine import Engine, EngineConfig

    return Engine.load(folder, EngineConfig(dtype=dtype, page_size=16, max_tokens=max_tokens, max_requests=4, poison_freed=True, **options))


def row_errors(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: the spread of the difference (its mean taken off) over the spread of the wanted logits."""
    difference = got - want
    difference = difference - difference.mean(axis=-1, keepdims=True)
    centred = want - want.mean(axis=-1, keepdims=True)
    return np.sqrt((difference**2).mean(axis=-1)) / np.sqrt((centred**2).mean())


def run_schedule(engine, requests: dict[str, list[int]], schedule: list[list[tuple[str, int]]]) -> dict[str, np.ndarray]:
    """Feeds the requests' tokens in the schedule's portions (every step one batch), asks for every position's logits,
    ends a request with its last token, and checks the cache's books after every step."""
    from lalamo_b200.engine.executor import StepEntry

    done = {name: 0 for name in requests}
    rows: dict[str, list[np.ndarray]] = {name: [] for name in requests}
    for step in schedule:
        entries = []
        for name, count in step:
            if done[name] == 0:
                engine.admit(name)
            entries.append(StepEntry(name, requests[name][done[name] : done[name] + count], list(range(count))))
        logits = engine.step(entries).float().cpu().numpy()
        offset = 0
        for name, count in step:
            rows[name].append(logits[offset : offset + count])
            offset += count
            done[name] += count
            if done[name] == len(requests[name]):
                engine.release(name)
        engine.executor.check_status()
        engine.cache.check()
    assert all(done[name] == len(tokens) for name, tokens in requests.items())
    return {name: np.concatenate(parts) for name, parts in rows.items()}


def close_enough(got: np.ndarray, want: np.ndarray, dtype: str) -> bool:
    """32-bit: every row within the limit.  bfloat16: the rounding of a router's input can turn a close call between two
    experts, which no limit on rounding errors covers, and random weights make a few close calls in a hundred tokens; so
    nine rows in ten must be within the limit and, where there are rows enough for one to mean something, the median
    within half of it.  (The kernels' edges are tested row by row in bfloat16 too, further down, where nothing is routed.)"""
    errors = row_errors(got, want)
    if dtype == "float32":
        return bool(errors.max() < FLOAT32_LIMIT)
    return bool(np.quantile(errors, 0.9) < BFLOAT16_LIMIT and (errors.size < 8 or np.median(errors) < BFLOAT16_LIMIT / 2))


# ----------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_a_prompt_at_once_and_token_by_token(models, name, dtype):
    folder, weights = models[name]
    config = CONFIGS[name]
    tokens = tokens_for(config, 90, 5)
    want = plain.forward(tokens, weights, config)
    engine = load_engine(folder, dtype)
    whole = run_schedule(engine, {"a": tokens}, [[("a", len(tokens))]])["a"]
    assert close_enough(whole, want, dtype)
    # the first 21 at once, the rest one by one: every window passes over decoded tokens, steps replay from recordings
    decoded = run_schedule(engine, {"b": tokens}, [[("b", 21)]] + [[("b", 1)]] * (len(tokens) - 21))["b"]
    assert close_enough(decoded, want, dtype)
    # from the very first token on, one by one
    single = run_schedule(engine, {"c": tokens[:40]}, [[("c", 1)]] * 40)["c"]
    assert close_enough(single, want[:40], dtype)
    assert engine.cache.free_pages() == engine.cache.num_pages


def test_the_stream_after_every_layer_run(models):
    """The 32-bit stream after every run of a layer (a repeated layer counts each time) against the plain implementation's."""
    folder, weights = models["A"]
    config = CONFIGS["A"]
    tokens = tokens_for(config, 30, 8)
    wanted: list[np.ndarray] = []
    plain.forward(tokens, weights, config, wanted)
    engine = load_engine(folder, "float32", cuda_graphs=False)
    seen: list[torch.Tensor] = []
    for block in engine.model.blocks:
        def tapped(residual, pending, step, cache, inner=block.forward):
            result = inner(residual, pending, step, cache)
            assert result is None   # the block has added everything
            seen.append(residual.clone())
            return result
        block.forward = tapped
    run_schedule(engine, {"a": tokens}, [[("a", len(tokens))]])
    assert len(seen) == len(wanted) == 8
    for index, (got, want) in enumerate(zip(seen, wanted)):
        assert np.abs(got.cpu().numpy() - want).max() < 2e-4 * np.abs(want).max(), index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_every_size(models, name, dtype):
    folder, weights = models[name]
    config = CONFIGS[name]
    tokens = tokens_for(config, 150, 6)
    want = plain.forward(tokens, weights, config)
    engine = load_engine(folder, dtype)
    for cuts in ([2, 3, 2, 5, 1, 17, 1, 1, 33, 2, 16, 31, 36], [64, 2, 2, 2, 48, 32], [7] * 21 + [3], [1, 2, 147]):
        assert sum(cuts) == len(tokens)
        got = run_schedule(engine, {"a": tokens}, [[("a", count)] for count in cuts])["a"]
        assert close_enough(got, want, dtype), cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype):
    """Up to four live requests of unequal lengths, portions beside single tokens; requests end and others take their
    slots and pages (which were overwritten with NaN when they were given back); a pool smaller than the sum."""
    folder, weights = models[name]
    config = CONFIGS[name]
    lengths = {"a": 70, "b": 1, "c": 33, "d": 2, "e": 95, "f": 18, "g": 64}
    requests = {key: tokens_for(config, count, 10 + index) for index, (key, count) in enumerate(lengths.items())}
    schedule = [
        [("a", 30), ("b", 1), ("c", 2)],
        [("a", 1), ("c", 1), ("d", 1), ("e", 17)],
        [("a", 1), ("c", 14), ("d", 1), ("e", 1)],
        [("a", 16), ("c", 1), ("e", 40), ("f", 3)],
        [("a", 1), ("c", 15), ("e", 1), ("f", 15)],
        [("a", 21), ("e", 2), ("g", 33)],
        [("e", 33), ("g", 1)],
        [("e", 1), ("g", 30)],
    ]
    engine = load_engine(folder, dtype, max_tokens=288)
    got = run_schedule(engine, requests, schedule)
    for key, tokens in requests.items():
        assert close_enough(got[key], plain.forward(tokens, weights, config), dtype), key
    # each request alone, in one piece, on the same engine: what the batch and the cutting change is rounding
    for key in ("a", "e"):
        alone = run_schedule(engine, {key: requests[key]}, [[(key, len(requests[key]))]])[key]
        assert row_errors(got[key], alone).max() < 5e-5 if dtype == "float32" else close_enough(got[key], alone, dtype), key
    assert engine.cache.free_pages() == engine.cache.num_pages


@pytest.mark.parametrize("name", ["A", "C"])
def test_windows_give_pages_back(models, name):
    """A request several times as long as the pool runs in portions, since its windows free the pages they have passed."""
    folder, weights = models[name]
    config = CONFIGS[name]
    tokens = tokens_for(config, 330, 21)
    want = plain.forward(tokens, weights, config)
    engine = load_engine(folder, "float32", max_tokens=96)
    schedule = [[("a", 16)]] * 15 + [[("a", 7)]] + [[("a", 1)]] * 83
    got = run_schedule(engine, {"a": tokens}, schedule)["a"]
    assert row_errors(got, want).max() < FLOAT32_LIMIT


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    folder, weights = models["C"]
    config = CONFIGS["C"]
    tokens = tokens_for(config, 420, 22)
    want = plain.forward(tokens, weights, config)
    engine = load_engine(folder, dtype)
    got = run_schedule(engine, {"a": tokens}, [[("a", 4)]] + [[("a", 1)]] * 416)["a"]
    assert close_enough(got, want, dtype) and close_enough(got[-50:], want[-50:], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_beside_a_short_request(models, dtype):
    folder, weights = models["C"]
    config = CONFIGS["C"]
    requests = {"a": tokens_for(config, 1300, 41), "b": tokens_for(config, 30, 42)}
    schedule = [[("a", 700), ("b", 5)], [("a", 1), ("b", 20)], [("a", 590), ("b", 1)], [("b", 4), ("a", 9)]]
    engine = load_engine(folder, dtype, max_tokens=2048)
    got = run_schedule(engine, requests, schedule)
    for key, tokens in requests.items():
        assert close_enough(got[key], plain.forward(tokens, weights, config), dtype), key


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(models, name):
    from lalamo_b200 import GenerationConfig, LanguageModel

    folder, weights = models[name]
    config = CONFIGS[name]
    model = LanguageModel.load(folder, dtype="float32", max_tokens=1024, max_requests=4)
    prompts = [tokens_for(config, count, 30 + count) for count in (1, 9, 30, 47, 2, 18)]
    produced = model.generate_tokens(prompts, GenerationConfig(temperature=0.0), max_output_length=12, eos_token_ids=[])
    compared = 0
    for prompt, generated in zip(prompts, produced):
        assert len(generated) == 12
        sequence = list(prompt)
        for token in generated:
            logits = plain.forward(sequence, weights, config)[-1]
            best = np.sort(logits)[-2:]
            if best[1] - best[0] < 1e-4:
                break   # a tie within 32-bit rounding: either token is right, and what follows depends on it
            assert token == int(np.argmax(logits))
            sequence.append(token)
        else:
            compared += 1
    assert compared >= 4   # sequences compared to their end
    model.engine.executor.check_status()
    assert model.engine.cache.free_pages() == model.engine.cache.num_pages


def test_command_line_and_step_replay(models, tmp_path):
    """The same model through the two programs a user runs: `generate` (greedy ids of the plain implementation) and the
    step replay that writes logits (portions, two live requests, a request that ends and another in its slot)."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    from trace_client import TraceRun

    root = Path(__file__).resolve().parent.parent
    folder, weights = models["B"]
    config = CONFIGS["B"]
    prompt = tokens_for(config, 11, 77)
    prompt_file = tmp_path / "prompts.txt"
    prompt_file.write_text(" ".join(str(token) for token in prompt) + "\n")
    command = [sys.executable, "-m", "lalamo_b200", "generate", str(folder), "--prompt-ids-file", str(prompt_file), "--max-tokens", "5", "--temperature", "0",
               "--dtype", "float32", "--max-cache-tokens", "256"]
    result = subprocess.run(command, cwd=root, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr
    produced = [json.loads(line) for line in result.stdout.splitlines() if line.startswith("{")][0]["token_ids"]
    sequence = list(prompt)
    for token in produced:
        logits = plain.forward(sequence, weights, config)[-1]
        best = np.sort(logits)[-2:]
        if best[1] - best[0] < 1e-4:
            break
        assert token == int(np.argmax(logits))
        sequence.append(token)

    requests = {name: tokens_for(config, count, 80 + count) for name, count in (("a", 40), ("b", 9), ("c", 21))}
    wanted = {name: plain.forward(tokens, weights, config) for name, tokens in requests.items()}
    run = TraceRun(folder, "float32", tmp_path / "out", 128, config["vocab"])
    steps = [([("a", 0, 17), ("b", 0, 2)], []), ([("a", 17, 18), ("b", 2, 9)], ["b"]), ([("a", 18, 40), ("c", 0, 21)], ["a", "c"])]
    for entries, ended in steps:
        got = run.step([{"id": name, "tokens": requests[name][lo:hi], "want": list(range(hi - lo))} for name, lo, hi in entries], ended)
        want = np.concatenate([wanted[name][lo:hi] for name, lo, hi in entries])
        assert row_errors(got, want).max() < FLOAT32_LIMIT
    assert run.close() == 0


# ---------------------------------------------------------------------- mechanisms alone
def as_int(values) -> torch.Tensor:
    return torch.tensor(list(values), dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,dim", [(37, 200), (5, 64), (300, 1024)])
def test_exact_norm_and_the_two_norms_in_one_kernel(rows, dim, dtype):
    from lalamo_b200 import ops

    generator = np.random.default_rng(rows)
    make = lambda *shape: torch.from_numpy(generator.standard_normal(shape))
    stream, a, b = 3 * make(rows, dim).float(), make(rows, dim).to(dtype), make(rows, dim).to(dtype)
    w_out, w_next = (0.2 * make(dim)).float(), (0.2 * make(dim)).float()
    eps = 1e-5
    out = torch.empty(rows, dim, dtype=dtype, device="cuda")
    ops.rmsnorm(stream.cuda(), w_out.cuda(), out, eps, scale_offset=1.0, exact=True)
    want = plain.offset_norm(stream.double().numpy(), w_out.double().numpy(), eps)
    tolerance = 1e-5 if dtype == torch.float32 else 2.0 ** -8
    assert (np.abs(out.float().cpu().numpy() - want) <= tolerance * np.maximum(1.0, np.abs(want))).all()   # one rounding
    # stream += norm(a + b); next = norm'(stream), one kernel
    device_stream = stream.cuda()
    following = torch.empty(rows, dim, dtype=dtype, device="cuda")
    ops.norm_accumulate(device_stream, ops.ScaledSum([(a.cuda(), 1.0, None), (b.cuda(), 1.0, None)]), w_out.cuda(), eps, scale_offset=1.0, rounded=following,
                        next_norm=(w_next.cuda(), eps, 1.0))
    new = stream.double().numpy() + plain.offset_norm(a.double().numpy() + b.double().numpy(), w_out.double().numpy(), eps)
    assert np.abs(device_stream.cpu().numpy() - new).max() < 1e-5
    want = plain.offset_norm(new, w_next.double().numpy(), eps)
    assert (np.abs(following.float().cpu().numpy() - want) <= tolerance * np.maximum(1.0, np.abs(want))).all()


def test_embedding_added_again_and_scaled_logits():
    from lalamo_b200 import ops

    generator = np.random.default_rng(4)
    table = torch.from_numpy(generator.standard_normal((50, 72))).to(torch.bfloat16)
    ids = [3, 49, 0, 3, 17]
    stream = torch.from_numpy(generator.standard_normal((5, 72))).float()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    device_stream = stream.cuda()
    ops.embed(table.cuda(), as_int(ids), device_stream, 4.0, status, accumulate=True)
    assert torch.allclose(device_stream.cpu(), stream + 4.0 * table.float()[ids], atol=1e-6)
    ops.scale_(device_stream, 0.25)
    assert torch.allclose(device_stream.cpu(), 0.25 * (stream + 4.0 * table.float()[ids]), atol=1e-6) and int(status.item()) == 0


@pytest.mark.parametrize("experts,top", [(8, 2), (6, 3), (4, 4), (5, 1), (64, 6), (33, 3)])
def test_router_with_a_bias_and_the_softmax_over_the_chosen(experts, top):
    from lalamo_b200 import ops

    generator = np.random.default_rng(experts + top)
    width, tokens = 96, 77
    x = torch.from_numpy(generator.standard_normal((tokens, width))).float()
    w = {"r.router": generator.standard_normal((experts, width)) * 0.3, "r.router.b": generator.standard_normal(experts)}
    router, bias = torch.from_numpy(w["r.router"]).float(), torch.from_numpy(w["r.router.b"]).float()
    w = {"r.router": router.double().numpy(), "r.router.b": bias.double().numpy()}
    chosen, weights = ops.moe_route(x.cuda(), router.cuda(), top=top, score="logits", bias=bias.cuda(), chosen_softmax=True)
    want_chosen, want_weights = plain.route(x.double().numpy(), w, "r.", top)
    assert (chosen.cpu().numpy() == want_chosen).all()
    assert np.abs(weights.cpu().numpy() - want_weights).max() < 1e-5
    # the bias decides: one that lifts the last expert above everything puts it first for every token
    bias[-1] = 100.0
    chosen, weights = ops.moe_route(x.cuda(), router.cuda(), top=top, score="logits", bias=bias.cuda(), chosen_softmax=True)
    assert (chosen[:, 0] == experts - 1).all() and (weights[:, 0] > 0.999).all() or top == experts


@pytest.mark.parametrize("path,dtype", [("plain", torch.float32), ("plain", torch.bfloat16), ("stream", torch.float32), ("stream", torch.bfloat16),
                                        ("grouped", torch.bfloat16), (None, torch.bfloat16)])
@pytest.mark.parametrize("tokens,width,ff,experts,top,limit", [(1, 72, 40, 6, 3, 1.0), (5, 72, 40, 6, 3, 0.5), (150, 72, 40, 6, 3, 2.0), (333, 256, 200, 9, 2, 1.5)])
def test_experts_with_the_limited_sigmoid_gate(tokens, width, ff, experts, top, limit, path, dtype):
    """Every way the experts' products are computed, with sums large enough that both limits bite."""
    from lalamo_b200 import ops

    generator = np.random.default_rng(tokens)
    make = lambda *shape: torch.from_numpy(generator.standard_normal(shape)).to(dtype)
    x, gate, up, down = make(tokens, width), make(experts, ff, width) / 6, make(experts, ff, width) / 6, make(experts, width, ff) / 6
    chosen = torch.from_numpy(np.stack([generator.permutation(experts - 1)[:top] for _ in range(tokens)]).astype(np.int32))
    weights = torch.from_numpy(generator.random((tokens, top))).float()
    got = ops.moe_experts(x.cuda(), gate.cuda(), up.cuda(), down.cuda(), chosen.cuda(), weights.cuda(), "sigmoid_limit", path=path, limit=limit)
    got = got.float().cpu().numpy()
    want = np.zeros((tokens, width))
    hit = 0
    for t in range(tokens):
        for e, s in zip(chosen[t].tolist(), weights[t].double().numpy()):
            w = {"gate": gate[e].double().numpy(), "up": up[e].double().numpy(), "down": down[e].double().numpy()}
            h = x[t : t + 1].double().numpy()
            hit += int((np.abs(h @ w["up"].T) > limit).sum() + (h @ w["gate"].T > limit).sum())
            want[t] += s * plain.expert(h, w, "", limit)[0]
    assert hit > 0
    assert np.abs(got - want).max() < (1e-4 if dtype == torch.float32 else 0.04) * np.abs(want).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,width,ff", [(3, 64, 40), (16, 128, 256), (17, 128, 256), (100, 128, 72), (200, 256, 320), (40, 72, 28), (600, 512, 520), (2048, 256, 1152)])
def test_dense_expert_with_the_limited_sigmoid_gate(tokens, width, ff, dtype):
    """The shared expert through the feed-forward part: few tokens (the weight-streaming product's epilogue), some (the one-tile
    tcgen05 product's) and many (the walking product's, with and without bulk stores)."""
    from lalamo_b200.config.plan import GatedMLPSpec
    from lalamo_b200.parts.base import Runtime, build_part

    generator = np.random.default_rng(tokens + ff)
    make = lambda *shape: torch.from_numpy(generator.standard_normal(shape)).to(dtype)
    w = {"gate": make(ff, width) / 4, "up": make(ff, width) / 4, "down": make(width, ff) / 6}
    x = make(tokens, width)
    part = build_part(GatedMLPSpec(model_dim=width, hidden_dim=ff, activation="sigmoid_limit", limit=1.25),
                      {"gate_proj": w["gate"], "up_proj": w["up"], "down_proj": w["down"]}, Runtime(torch.device("cuda"), dtype))
    got = part.forward(x.cuda())
    if not isinstance(got, torch.Tensor):
        got = got.sum()
    want = plain.expert(x.double().numpy(), {name: tensor.double().numpy() for name, tensor in w.items()}, "", 1.25)
    assert np.abs(got.float().cpu().numpy() - want).max() < (1e-4 if dtype == torch.float32 else 0.04) * np.abs(want).max()


def latent_rows_in_pages(rows: np.ndarray, page_size: int, dtype: torch.dtype, seed: int):
    """Rows ``[n, latent + rope]`` of one request laid out in shuffled pages among NaN."""
    n, full = rows.shape
    blocks = -(-n // page_size)
    num_pages = blocks + 5
    order = np.random.default_rng(seed).permutation(num_pages)[:blocks]
    pages = torch.full((num_pages, page_size, 1, full), float("nan"), dtype=dtype, device="cuda")
    source = torch.from_numpy(rows).to(dtype).cuda()
    for block, page in enumerate(order.tolist()):
        count = min(page_size, n - block * page_size)
        pages[page, :count, 0] = source[block * page_size : block * page_size + count]
    return pages, as_int(order.tolist()).reshape(1, -1)


def plain_latent_sums(q: np.ndarray, rows: np.ndarray, positions, latent: int, scale: float, window: int) -> np.ndarray:
    out = np.zeros((len(positions), q.shape[1], latent))
    for index, p in enumerate(positions):
        first = max(0, p - window + 1)
        seen = rows[first : p + 1]
        for head in range(q.shape[1]):
            scores = seen @ q[index, head] * scale
            weights = np.exp(scores - scores.max())
            out[index, head] = (weights / weights.sum()) @ seen[:, :latent]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("latent,rope,heads", [(64, 32, 4), (40, 12, 3), (128, 64, 2), (24, 2, 1)])
def test_latent_attention_edges_with_one_row_that_stands_out(latent, rope, heads, dtype):
    """One row among hundreds carries almost all the weight where it is seen: queries for which it lies just inside and just
    outside the window, at page borders, at the very start, and far back."""
    from lalamo_b200 import ops

    generator = np.random.default_rng(latent + rope)
    n, page_size, window, full = 400, 16, 37, latent + rope
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for special in (0, 1, 15, 16, 200, 223, 224, 362):
        rows = 0.3 * generator.standard_normal((n, full))
        direction = generator.standard_normal(full)
        direction[0] = 0.0
        direction /= np.linalg.norm(direction)
        rows[special] = 6.0 * direction
        rows[special, 0] = 30.0   # what it adds to the sum shows in channel 0, which no query looks at
        positions = sorted({p for p in (special, special + 1, special + window - 2, special + window - 1, special + window, special + window + 1,
                                        special + 2 * page_size, n - 1, 15, 16, 17) if special <= p < n} | {0, 1})
        q = 0.3 * generator.standard_normal((len(positions), heads, full)) + 4.0 * direction
        q[..., 0] = 0.0
        rows = torch.from_numpy(rows).to(dtype).double().numpy()
        q = torch.from_numpy(q).to(dtype).double().numpy()
        want = plain_latent_sums(q, rows, positions, latent, 0.5, window)
        pages, table = latent_rows_in_pages(rows, page_size, dtype, special)
        out = torch.empty(len(positions), heads, latent, dtype=dtype, device="cuda")
        ops.latent_attention_plain(torch.from_numpy(q).to(dtype).cuda().contiguous(), pages, out, positions=as_int(positions),
                                   token_segment=torch.zeros(len(positions), dtype=torch.int32, device="cuda"), block_table=table, num_heads=heads,
                                   latent=latent, rope=rope, scale=0.5, window=window, status=status)
        got = out.float().cpu().numpy()
        assert int(status.item()) == 0
        assert np.abs(got - want).max() < (1e-3 if dtype == torch.float32 else 0.3), special
        inside = positions.index(special + window - 1) if special + window - 1 < n else None
        if inside is not None and special + window < n:   # the edge itself: seen by the last query of its window, gone for the next
            assert want[inside, :, 0].min() > 25 and np.abs(want[positions.index(special + window)]).max() < 5


@pytest.mark.parametrize("splits", [1, 3, 32])
@pytest.mark.parametrize("latent,rope,heads,window,special", [(64, 32, 4, 37, 100), (128, 64, 8, 150, 249), (256, 32, 16, 64, 0), (32, 16, 3, 1, 7), (144, 48, 5, 300, 63),
                                                             (64, 0, 70, 129, 130)])
def test_tensor_core_latent_attention_at_every_position(latent, rope, heads, window, special, splits):
    """Every position of a 400-token request as a query on the tensor-core kernel, in one portion and cut into portions that
    start anywhere (runs of tokens shorter than a CTA takes, single tokens), with the cached rows shared out over CTAs or not;
    one row stands out wherever it is seen."""
    from lalamo_b200 import ops

    generator = np.random.default_rng(latent + window)
    n, page_size, full, dtype = 400, 16, latent + rope, torch.bfloat16
    rows = 0.3 * generator.standard_normal((n, full))
    direction = generator.standard_normal(full)
    direction[0] = 0.0
    direction /= np.linalg.norm(direction)
    rows[special] = 6.0 * direction
    rows[special, 0] = 30.0
    q = 0.3 * generator.standard_normal((n, heads, full)) + 4.0 * direction
    q[..., 0] = 0.0
    rows, q = (torch.from_numpy(a).to(dtype).double().numpy() for a in (rows, q))
    want = plain_latent_sums(q, rows, list(range(n)), latent, 0.5, window)
    pages, table = latent_rows_in_pages(rows, page_size, dtype, special)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    run = ops.latent_attention_tiling(heads)[1]
    for portions in ([n], [1, 2, 3, 64, 1, 1, 100, 29, 199]):
        out = torch.zeros(n, heads, latent, dtype=dtype, device="cuda")
        starts = np.concatenate([[0], np.cumsum(portions)[:-1]])
        items = [(first, min(run, start + length - first)) for start, length in zip(starts, portions) for first in range(start, start + length, run)]
        ops.latent_attention(torch.from_numpy(q).to(dtype).cuda().contiguous(), pages, out, items=as_int(np.asarray(items).reshape(-1)), num_items=len(items),
                             positions=torch.arange(n, dtype=torch.int32, device="cuda"), token_segment=torch.zeros(n, dtype=torch.int32, device="cuda"),
                             block_table=table, num_heads=heads, latent=latent, rope=rope, scale=0.5, window=window, status=status, splits=splits)
        got = out.float().cpu().numpy()
        assert int(status.item()) == 0
        worst = np.abs(got - want).max(axis=(1, 2))
        assert worst.max() < 0.3, (portions, int(worst.argmax()), float(worst.max()))
    if special + window < n:
        assert want[special + window - 1, :, 0].min() > 25 and np.abs(want[special + window]).max() < 5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_rows_and_queries_are_prepared_as_the_plain_implementation_does(dtype):
    """Norm of the latent, rotation of the shared key part and of the queries' rotated parts, written through a block table;
    inputs are column slices of one wider product."""
    from lalamo_b200 import ops

    generator = np.random.default_rng(9)
    tokens, heads, dim, rope, latent, page_size = 21, 3, 10, 6, 20, 4
    q_width = heads * (dim + rope)
    product = torch.from_numpy(generator.standard_normal((tokens, q_width + 7 + latent + rope))).to(dtype)
    q_latent = torch.from_numpy(generator.standard_normal((heads, tokens, latent))).to(dtype)
    weight = torch.from_numpy(1 + 0.2 * generator.standard_normal(latent)).float()
    positions = [5, 6, 7, 8, 9, 10, 11, 12, 13, 0, 1, 2, 3, 4, 100, 101, 102, 103, 104, 105, 106]
    segments = [0] * 9 + [1] * 5 + [2] * 7
    blocks = 27
    table = torch.full((3, blocks), -1, dtype=torch.int32)
    table[0, :4] = torch.tensor([3, 9, 1, 0])
    table[1, :2] = torch.tensor([4, 7])
    table[2, 25:27] = torch.tensor([8, 2])
    pages = torch.full((10, page_size, 1, latent + rope), float("nan"), dtype=dtype, device="cuda")
    queries = torch.empty(tokens, heads, latent + rope, dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    device_product = product.cuda()
    inv_freq = torch.tensor([50.0 ** (-2.0 * i / rope) for i in range(rope // 2)], dtype=torch.float32, device="cuda")
    ops.latent_prepare(device_product[:, :q_width], q_latent.cuda(), device_product[:, q_width + 7 :], queries, pages, norm_weight=weight.cuda(), eps=1e-5,
                       scale_offset=0.0, inv_freq=inv_freq, positions=as_int(positions), token_segment=as_int(segments), block_table=table.cuda(),
                       num_heads=heads, head_dim=dim, latent=latent, rope=rope, write_kv=True, status=status)
    assert int(status.item()) == 0
    x = product.double().numpy()
    down = x[:, q_width + 7 :]
    want_latent = plain.rms_norm(down[:, :latent], weight.double().numpy(), 1e-5)
    want_key = plain.rotate_half(down[:, None, latent:], np.asarray(positions), rope, 50.0)[:, 0]
    want_q = plain.rotate_half(x[:, :q_width].reshape(tokens, heads, dim + rope)[..., dim:], np.asarray(positions), rope, 50.0)
    tolerance = 1e-5 if dtype == torch.float32 else 0.03
    host_pages = pages.float().cpu().numpy()
    for token, (position, segment) in enumerate(zip(positions, segments)):
        row = host_pages[int(table[segment, position // page_size]), position % page_size, 0]
        assert np.abs(row[:latent] - want_latent[token]).max() < tolerance and np.abs(row[latent:] - want_key[token]).max() < tolerance
    got = queries.float().cpu().numpy()
    assert np.abs(got[..., latent:] - want_q).max() < tolerance
    assert np.array_equal(got[..., :latent], q_latent.float().numpy().transpose(1, 0, 2))
    assert np.isnan(host_pages[5]).all() and np.isnan(host_pages[6]).all()   # pages of nobody stay untouched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_heads_products_and_the_gate(dtype):
    from lalamo_b200 import ops

    generator = np.random.default_rng(12)
    heads, tokens, k, n = 3, 19, 24, 40
    wide = torch.from_numpy(generator.standard_normal((tokens, heads, k + 5))).to(dtype).cuda()
    weight = torch.from_numpy(generator.standard_normal((heads, k, n)) / 5).to(dtype).cuda()
    got = ops.heads_linear(wide[:, :, :k].transpose(0, 1), weight)
    want = np.einsum("thk,hkn->htn", wide[:, :, :k].double().cpu().numpy(), weight.double().cpu().numpy())
    assert got.shape == (heads, tokens, n) and got.is_contiguous()
    assert np.abs(got.float().cpu().numpy() - want).max() < (1e-4 if dtype == torch.float32 else 0.05)
    back = ops.heads_linear(got, weight, transpose_weight=True)
    assert back.shape == (heads, tokens, k)
    gate = torch.from_numpy(generator.standard_normal((tokens, heads * n + 3))).to(dtype).cuda()
    mixed = torch.empty(tokens, heads * n, dtype=dtype, device="cuda")
    ops.gate_heads(got, gate[:, 3:], mixed)
    want = got.double().cpu().numpy().transpose(1, 0, 2).reshape(tokens, heads * n) * plain.sigmoid(gate[:, 3:].double().cpu().numpy())
    assert np.abs(mixed.float().cpu().numpy() - want).max() < (1e-5 if dtype == torch.float32 else 0.03)


@pytest.mark.parametrize("tokens,heads,k,n", [(19, 3, 48, 80), (64, 2, 64, 256), (150, 5, 256, 64), (1, 16, 64, 128), (300, 1, 16, 16), (8, 4, 128, 512)])
def test_heads_products_of_the_frameworks_own(tokens, heads, k, n):
    """The per-head products on the framework's kernel: both orientations of the heads' matrices, inputs that are column slices of wider
    rows, outputs that are parts of wider rows, the gate read from a slice; token counts that fill no block of 64."""
    from lalamo_b200 import ops

    generator = np.random.default_rng(tokens + k)
    make = lambda *shape: torch.from_numpy(generator.standard_normal(shape)).to(torch.bfloat16).cuda()
    wide = make(tokens, heads * (k + 8) + 24)   # heads of k + 8 channels of which the first k are used, then other columns
    x = wide[:, : heads * (k + 8)].view(tokens, heads, k + 8)[:, :, :k]
    w_kn = make(heads, k, n) / 4
    out_wide = torch.full((tokens, heads, n + 16), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.heads_product(x, w_kn, out_wide[:, :, :n], weight_is_kn=True)
    want = np.einsum("thk,hkn->thn", x.double().cpu().numpy(), w_kn.double().cpu().numpy())
    assert np.abs(out_wide[:, :, :n].float().cpu().numpy() - want).max() < 0.02 * max(1.0, np.abs(want).max())
    assert (out_wide[:, :, n:] == 7.0).all()   # the rest of the rows stays
    w_nk = make(heads, n, k) / 4
    gate_wide = make(tokens, 10 + heads * n)
    gate = gate_wide[:, 10:].view(tokens, heads, n)
    out = torch.empty(tokens, heads * n, dtype=torch.bfloat16, device="cuda")
    ops.heads_product(x, w_nk, out.view(tokens, heads, n), weight_is_kn=False, gate=gate)
    want = np.einsum("thk,hnk->thn", x.double().cpu().numpy(), w_nk.double().cpu().numpy()) * plain.sigmoid(gate.double().cpu().numpy())
    assert np.abs(out.view(tokens, heads, n).float().cpu().numpy() - want).max() < 0.02 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_norm_kernel_adds_the_experts_outputs_itself(dtype):
    """The experts' weighted sum left to the norm kernel (pairs without an expert hold NaN and count nothing) beside a second term."""
    from lalamo_b200 import ops

    generator = np.random.default_rng(31)
    rows, dim, top, experts = 23, 200, 3, 5
    make = lambda *shape: torch.from_numpy(generator.standard_normal(shape))
    stream, shared = make(rows, dim).float(), make(rows, dim).to(dtype)
    pair_out, weights = make(rows * top, dim).float(), torch.from_numpy(generator.random((rows, top))).float()
    chosen = torch.from_numpy(generator.integers(0, experts, size=(rows, top)).astype(np.int32))
    chosen[4, 1] = experts   # no expert
    pair_out[4 * top + 1] = float("nan")
    weight, following = (0.2 * make(dim)).float(), (0.2 * make(dim)).float()
    used = pair_out.double().reshape(rows, top, dim).clone()
    used[4, 1] = 0.0
    routed = (weights.double()[:, :, None] * used).sum(1)
    total = routed.numpy() + shared.double().numpy()
    new = stream.double().numpy() + plain.offset_norm(total, weight.double().numpy(), 1e-6)
    term = ops.ExpertSum(pair_out.cuda(), weights.cuda(), chosen.cuda(), experts, dtype)
    device_stream = stream.cuda()
    normed = torch.empty(rows, dim, dtype=dtype, device="cuda")
    ops.norm_accumulate(device_stream, ops.ScaledSum([(term, 1.0, None), (shared.cuda(), 1.0, None)]), weight.cuda(), 1e-6, scale_offset=1.0, rounded=normed,
                        next_norm=(following.cuda(), 1e-6, 1.0))
    assert np.abs(device_stream.cpu().numpy() - new).max() < 1e-5
    want = plain.offset_norm(new, following.double().numpy(), 1e-6)
    assert np.abs(normed.float().cpu().numpy() - want).max() < (1e-5 if dtype == torch.float32 else 0.02)
    # the same sum as a plain tensor, and through the two terms' plain sum
    assert np.abs(term.sum().float().cpu().numpy() - routed.numpy()).max() < (1e-5 if dtype == torch.float32 else 0.03)
    both = ops.ScaledSum([(term, 1.0, None), (shared.cuda(), 1.0, None)]).sum()
    assert np.abs(both.float().cpu().numpy() - total).max() < (1e-5 if dtype == torch.float32 else 0.05)
