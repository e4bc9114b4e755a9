"""The Vuvulorn design on the GPU against the plain NumPy restatement (``plain_vuvulorn.py``): each mechanism's
kernels alone, then whole models through the engine: prompts at once, decoding through the cache, portions of
every size, mixed batches with pages and state slots that are freed and used again, window and kept-token edges,
long decoding, and greedy generation through the Python entry point."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_vuvulorn as plain
from tiny_vuvulorn import CONFIGS, write_model

pytestmark = pytest.mark.gpu

FLOAT32_LIMIT = 2e-4   # of the logits' spread; 32-bit sums of a few hundred terms stay far below
BFLOAT16_LIMIT = 0.08


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("vuvulorn")
    return {name: write_model(root / name, config, seed) for seed, (name, config) in enumerate(CONFIGS.items())}


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
    nine rows in ten must be within the limit and the median within half of it.  (The kernels' edges are tested row by
    row in bfloat16 too, further down, where nothing is routed.)"""
    errors = row_errors(got, want)
    if dtype == "float32":
        return bool(errors.max() < FLOAT32_LIMIT)
    return bool(np.quantile(errors, 0.9) < BFLOAT16_LIMIT and np.median(errors) < BFLOAT16_LIMIT / 2)


# ----------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_a_prompt_at_once_and_token_by_token(models, name, dtype):
    folder, weights = models[name]
    config = CONFIGS[name]
    tokens = tokens_for(config, 90, 5)
    want = plain.forward(config, weights, tokens)
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_portions_of_every_size(models, name, dtype):
    folder, weights = models[name]
    config = CONFIGS[name]
    tokens = tokens_for(config, 150, 6)
    want = plain.forward(config, weights, tokens)
    engine = load_engine(folder, dtype)
    for cuts in ([2, 3, 2, 5, 1, 17, 1, 1, 33, 2, 16, 31, 36], [64, 2, 2, 2, 48, 32], [7] * 21 + [3], [1, 2, 147]):
        assert sum(cuts) == len(tokens)
        got = run_schedule(engine, {"a": tokens}, [[("a", count)] for count in cuts])["a"]
        assert close_enough(got, want, dtype), cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
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
        want = plain.forward(config, weights, tokens)
        assert close_enough(got[key], want, dtype), key
    # each request alone, in one piece, on the same engine: what the batch and the cutting change is rounding
    for key in ("a", "e"):
        alone = run_schedule(engine, {key: requests[key]}, [[(key, len(requests[key]))]])[key]
        assert row_errors(got[key], alone).max() < 5e-5 if dtype == "float32" else close_enough(got[key], alone, dtype), key
    assert engine.cache.free_pages() == engine.cache.num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "R"])
def test_long_portions(models, name, dtype):
    """Portions long enough for the recurrence to run them as chunks side by side, beside a short request, then decoding."""
    folder, weights = models[name]
    config = CONFIGS[name]
    requests = {"a": tokens_for(config, 1900, 41), "b": tokens_for(config, 30, 42)}
    schedule = [[("a", 1000), ("b", 5)], [("a", 1), ("b", 20)], [("a", 890), ("b", 1)], [("b", 4), ("a", 9)]]
    engine = load_engine(folder, dtype, max_tokens=4096)
    got = run_schedule(engine, requests, schedule)
    for key, tokens in requests.items():
        assert close_enough(got[key], plain.forward(config, weights, tokens), dtype), key


def test_a_window_gives_pages_back_and_keeps_the_first_ones(models):
    """A request four times as long as the pool runs in portions, since its windows free the pages they have passed;
    the pages of the kept first tokens stay, and decoding goes on over them."""
    folder, weights = models["P"]
    config = CONFIGS["P"]
    tokens = tokens_for(config, 260, 21)
    want = plain.forward(config, weights, tokens)
    engine = load_engine(folder, "float32", max_tokens=64)
    schedule = [[("a", 16)]] * 12 + [[("a", 5)]] + [[("a", 1)]] * 63
    got = run_schedule(engine, {"a": tokens}, schedule)["a"]
    assert row_errors(got, want).max() < FLOAT32_LIMIT


def test_long_decoding(models):
    folder, weights = models["Q"]
    config = CONFIGS["Q"]
    tokens = tokens_for(config, 420, 22)
    want = plain.forward(config, weights, tokens)
    engine = load_engine(folder, "float32")
    got = run_schedule(engine, {"a": tokens}, [[("a", 4)]] + [[("a", 1)]] * 416)["a"]
    errors = row_errors(got, want)
    assert errors.max() < FLOAT32_LIMIT and errors[-50:].max() < FLOAT32_LIMIT


@pytest.mark.parametrize("name", ["P", "R"])
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
            logits = plain.forward(config, weights, sequence)[-1]
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
    folder, weights = models["Q"]
    config = CONFIGS["Q"]
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
        logits = plain.forward(config, weights, sequence)[-1]
        best = np.sort(logits)[-2:]
        if best[1] - best[0] < 1e-4:
            break
        assert token == int(np.argmax(logits))
        sequence.append(token)

    requests = {name: tokens_for(config, count, 80 + count) for name, count in (("a", 40), ("b", 9), ("c", 21))}
    wanted = {name: plain.forward(config, weights, tokens) for name, tokens in requests.items()}
    run = TraceRun(folder, "float32", tmp_path / "out", 128, config["vocab"])
    steps = [([("a", 0, 17), ("b", 0, 2)], []), ([("a", 17, 18), ("b", 2, 9)], ["b"]), ([("a", 18, 40), ("c", 0, 21)], ["a", "c"])]
    for entries, ended in steps:
        got = run.step([{"id": name, "tokens": requests[name][lo:hi], "want": list(range(hi - lo))} for name, lo, hi in entries], ended)
        want = np.concatenate([wanted[name][lo:hi] for name, lo, hi in entries])
        assert row_errors(got, want).max() < FLOAT32_LIMIT
    assert run.close() == 0


# ---------------------------------------------------------------------- mechanisms alone
def paged(keys: np.ndarray, values: np.ndarray, page_size: int, dtype: torch.dtype, seed: int):
    """Keys ``[n, groups, dim]`` and values ``[n, groups, vdim]`` of one request laid out in shuffled pages among NaN."""
    n, groups, dim = keys.shape
    vdim = values.shape[-1]
    blocks = -(-n // page_size)
    num_pages = blocks + 5
    order = np.random.default_rng(seed).permutation(num_pages)[:blocks]
    k_pages = torch.full((num_pages, page_size, groups, dim), float("nan"), dtype=dtype, device="cuda")
    v_pages = torch.full((num_pages, groups, vdim, page_size), float("nan"), dtype=dtype, device="cuda")
    for position in range(n):
        page = int(order[position // page_size])
        k_pages[page, position % page_size] = torch.from_numpy(keys[position]).to(dtype)
        v_pages[page, :, :, position % page_size] = torch.from_numpy(values[position]).to(dtype)
    table = torch.from_numpy(order.astype(np.int32)).reshape(1, -1).cuda()
    return k_pages, v_pages, table


def plain_masked_attention(q, keys, values, positions, scale, window, keep_first):
    """float64: query rows ``[m, heads, dim]`` at ``positions`` over keys ``[n, groups, dim]``."""
    m, heads, _ = q.shape
    n, groups, _ = keys.shape
    out = np.zeros((m, heads, values.shape[-1]))
    for row, position in enumerate(positions):
        j = np.arange(n)
        seen = (j <= position) & ((position - j < window) | (j < keep_first))
        for head in range(heads):
            g = head // (heads // groups)
            scores = np.where(seen, keys[:, g] @ q[row, head] * scale, -np.inf)
            p = np.exp(scores - scores.max())
            out[row, head] = (p / p.sum()) @ values[:, g]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,vdim", [(64, 64), (32, 48), (16, 8)])
def test_attention_edges_with_one_key_that_stands_out(dim, vdim, dtype):
    """One key among hundreds carries almost all the weight where it is seen: queries for which it lies just inside and
    just outside the window, among the kept first keys and just past them, at page borders, and far back."""
    from lalamo_b200 import ops

    generator = np.random.default_rng(dim + vdim)
    n, heads, groups, page_size, window = 400, 4, 2, 16, 37
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for keep_first, special in ((5, 4), (5, 5), (16, 15), (17, 16), (0, 0), (33, 200), (3, 223), (3, 224)):
        keys = 0.3 * generator.standard_normal((n, groups, dim))
        values = generator.standard_normal((n, groups, vdim))
        direction = generator.standard_normal(dim)
        direction /= np.linalg.norm(direction)
        keys[special] = 6.0 * direction
        values[special] = 50.0
        positions = sorted({p for p in (special, special + 1, special + window - 1, special + window, special + window + 1, special + 2 * page_size,
                                        keep_first, keep_first + window, n - 1, 15, 16, 17) if special <= p < n} | {0, 1})
        q = 0.3 * generator.standard_normal((len(positions), heads, dim)) + 4.0 * direction
        keys = torch.from_numpy(keys).to(dtype).double().numpy()
        values = torch.from_numpy(values).to(dtype).double().numpy()
        q = torch.from_numpy(q).to(dtype).double().numpy()
        want = plain_masked_attention(q, keys, values, positions, 0.5, window, keep_first)
        k_pages, v_pages, table = paged(keys, values, page_size, dtype, special)
        out = torch.empty(len(positions), heads * vdim, dtype=dtype, device="cuda")
        ops.paged_attention_plain(
            torch.from_numpy(q).to(dtype).cuda().reshape(len(positions), -1).contiguous(), k_pages, v_pages, out,
            positions=torch.tensor(positions, dtype=torch.int32, device="cuda"), token_segment=torch.zeros(len(positions), dtype=torch.int32, device="cuda"),
            block_table=table, num_heads=heads, num_groups=groups, head_dim=dim, scale=0.5, window=window, status=status, value_dim=vdim, keep_first=keep_first)
        got = out.float().cpu().numpy().reshape(want.shape)
        assert int(status.item()) == 0
        assert np.abs(got - want).max() < (1e-3 if dtype == torch.float32 else 0.5), (keep_first, special)


@pytest.mark.parametrize("kernel", ["alone", "tiles-mma", "tiles-tcgen05", "tiles-tcgen05-pairs"])
@pytest.mark.parametrize("dim", [64, 32])
@pytest.mark.parametrize("window,keep_first,special", [(37, 5, 4), (37, 5, 5), (37, 16, 15), (37, 17, 16), (37, 0, 100), (100, 70, 69), (100, 64, 64), (20, 130, 129),
                                                       (64, 1, 0), (1, 3, 2), (300, 40, 39)])
def test_tensor_core_attention_with_kept_first_keys(window, keep_first, special, dim, kernel):
    """Every position of a 400-token request as a query, on each of the tensor-core kernels: tokens that attend alone
    (keys split over CTAs) and tiles of consecutive tokens; one key stands out wherever it is seen."""
    from lalamo_b200 import ops

    if kernel.startswith("tiles-tcgen05") and dim != 64:
        pytest.skip("the tcgen05 attention takes head size 64")
    generator = np.random.default_rng(window + keep_first + special)
    n, heads, groups, page_size, dtype = 400, 4, 2, 16, torch.bfloat16
    keys = 0.3 * generator.standard_normal((n, groups, dim))
    values = generator.standard_normal((n, groups, dim))
    direction = generator.standard_normal(dim)
    direction /= np.linalg.norm(direction)
    keys[special] = 6.0 * direction
    values[special] = 50.0
    q = 0.3 * generator.standard_normal((n, heads, dim)) + 4.0 * direction
    keys, values, q = (torch.from_numpy(a).to(dtype).double().numpy() for a in (keys, values, q))
    positions = list(range(n))
    want = plain_masked_attention(q, keys, values, positions, 0.5, window, keep_first)
    k_pages, v_pages, table = paged(keys, values, page_size, dtype, special)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros(n, heads * dim, dtype=dtype, device="cuda")
    common = dict(positions=torch.arange(n, dtype=torch.int32, device="cuda"), token_segment=torch.zeros(n, dtype=torch.int32, device="cuda"), block_table=table,
                  num_heads=heads, num_groups=groups, head_dim=dim, scale=0.5, window=window, status=status, keep_first=keep_first)
    queries = torch.from_numpy(q).to(dtype).cuda().reshape(n, -1).contiguous()
    if kernel == "alone":
        ops.attention_decode(queries, k_pages, v_pages, out, max_context=n, **common)
    else:
        tiles = torch.tensor([[first, min(32, n - first)] for first in range(0, n, 32)], dtype=torch.int32, device="cuda").reshape(-1)
        ops.attention_prefill(queries, k_pages, v_pages, out, tiles=tiles, num_tiles=tiles.numel() // 2, kernel="mma" if kernel == "tiles-mma" else "tcgen05",
                              split_tiles=2 if kernel.endswith("pairs") else 0, **common)
    got = out.float().cpu().numpy().reshape(want.shape)
    assert int(status.item()) == 0
    worst = np.abs(got - want).max(axis=(1, 2))
    assert worst.max() < 0.5, (int(worst.argmax()), float(worst.max()))


LONG_STEPS = [{0: 3, 1: 1}, {0: 1000, 1: 20}, {0: 1, 1: 2}, {1: 14, 0: 769}, {0: 27}]   # portions long enough to run as chunks, a last chunk of one token


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,groups,dk,dv,taps,steps", [
    (2, 1, 16, 32, 3, None), (3, 3, 40, 24, 1, None), (2, 2, 72, 16, 4, None), (4, 2, 128, 64, 2, None), (1, 1, 160, 40, 3, None),
    (2, 1, 16, 32, 3, LONG_STEPS), (2, 2, 64, 128, 4, LONG_STEPS), (3, 1, 18, 40, 2, LONG_STEPS), (1, 1, 128, 72, 3, LONG_STEPS)])
def test_gated_delta_rule_in_portions_against_the_recurrence(heads, groups, dk, dv, taps, steps, dtype):
    """Two requests in different slots, cut differently, a far write that must survive hundreds of decays close to one;
    with long portions, which run as chunks side by side from zero states and are put together afterwards."""
    from lalamo_b200 import ops

    generator = np.random.default_rng(dk * dv + taps)
    channels = 2 * groups * dk + heads * dv
    lengths = {0: 150, 1: 37} if steps is None else {0: 1800, 1: 37}
    proj = {r: torch.from_numpy(generator.standard_normal((n, channels + heads))).to(dtype) for r, n in lengths.items()}
    low = {r: torch.from_numpy(generator.standard_normal((n, heads * (dk + dv)))).to(dtype) for r, n in lengths.items()}
    conv = torch.from_numpy(0.6 * generator.standard_normal((channels, taps))).float()
    a_log = torch.tensor(generator.standard_normal(heads) - 4.0).float()   # decays close to one: what was written far back stays
    dt_bias = torch.from_numpy(generator.standard_normal(heads * dk)).float()
    norm = torch.from_numpy(1 + 0.2 * generator.standard_normal(dv)).float()
    eps = 1e-5

    def wanted(r):
        x, lr = proj[r].double().numpy(), low[r].double().numpy()
        n = x.shape[0]
        mixed = plain.silu(plain.short_convolution(x[:, :channels], conv.double().numpy()))
        q = mixed[:, : groups * dk].reshape(n, groups, dk)
        k = mixed[:, groups * dk : 2 * groups * dk].reshape(n, groups, dk)
        v = mixed[:, 2 * groups * dk :].reshape(n, heads, dv)
        q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk**-0.5
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
        per = heads // groups
        beta = plain.sigmoid(x[:, channels:])
        g = np.exp(-np.exp(a_log.double().numpy())[None, :, None] * plain.softplus(lr[:, : heads * dk] + dt_bias.double().numpy()).reshape(n, heads, dk))
        o = plain.delta_rule(np.repeat(q, per, 1), np.repeat(k, per, 1), v, beta, g)
        return (plain.rms_norm(o, norm.double().numpy(), eps) * plain.sigmoid(lr[:, heads * dk :]).reshape(n, heads, dv)).reshape(n, heads * dv)

    slots = 3
    matrix_state = torch.full((slots, heads, dk, dv), float("nan"), device="cuda")
    conv_state = torch.full((slots, max(taps - 1, 1), channels), float("nan"), dtype=dtype, device="cuda")
    slot_of = {0: 2, 1: 0}
    for slot in slot_of.values():
        matrix_state[slot] = 0
        conv_state[slot] = 0
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    steps = steps or [{0: 3, 1: 1}, {0: 1, 1: 20}, {0: 64}, {1: 2, 0: 2}, {0: 17, 1: 14}, {0: 63}]
    done = {0: 0, 1: 0}
    got = {0: [], 1: []}
    for step in steps:
        order = list(step)
        rows = torch.cat([proj[r][done[r] : done[r] + step[r]] for r in order]).cuda().contiguous()
        lows = torch.cat([low[r][done[r] : done[r] + step[r]] for r in order]).cuda().contiguous()
        counts = [step[r] for r in order]
        starts = np.concatenate([[0], np.cumsum(counts)[:-1]])
        as_int = lambda values: torch.tensor(list(values), dtype=torch.int32, device="cuda")
        plan = ops.gated_delta_chunk_plan(starts.tolist(), counts)
        chunk_plan = {name: as_int(array.tolist()) for name, array in plan.items()}
        chunk_plan.update(num_chunks=plan["chunk_start"].size, num_long=plan["long_table"].size // 3, num_direct=plan["direct"].size)
        out = ops.gated_delta_rule(
            rows, lows, conv_state if taps > 1 else None, matrix_state, conv_weight=conv.cuda(), a_log=a_log.cuda(), dt_bias=dt_bias.cuda(), norm_weight=norm.cuda(),
            norm_eps=eps, num_heads=heads, num_groups=groups, key_dim=dk, value_dim=dv, unit_eps=1e-6, token_segment=as_int(np.repeat(np.arange(len(order)), counts)),
            segment_start=as_int(starts), segment_length=as_int(counts), segment_slot=as_int(slot_of[r] for r in order), segments=len(order), status=status,
            chunk_plan=chunk_plan)
        out = out.float().cpu().numpy()
        for r, start, count in zip(order, starts, counts):
            got[r].append(out[start : start + count])
            done[r] += count
    assert int(status.item()) == 0 and done == lengths
    assert torch.isnan(matrix_state[1]).all()   # the slot nobody holds was not touched
    for r in lengths:
        want = wanted(r)
        assert np.abs(np.concatenate(got[r]) - want).max() < (2e-4 if dtype == torch.float32 else 0.05) * max(1.0, np.abs(want).max()), r


@pytest.mark.parametrize("experts,top,count,keep", [(8, 2, 2, 1), (6, 2, 3, 2), (4, 4, 1, 1), (5, 1, 5, 2), (64, 6, 8, 3), (33, 3, 1, 1)])
def test_router_choice_and_weights(experts, top, count, keep):
    from lalamo_b200 import ops

    generator = np.random.default_rng(experts + top)
    width, tokens = 96, 77
    x = torch.from_numpy(generator.standard_normal((tokens, width))).float()
    router = torch.from_numpy(generator.standard_normal((experts, width)) * 0.3).float()
    chosen, weights = ops.moe_route(x.cuda(), router.cuda(), top=top, group_count=count, group_keep=keep)
    want_chosen, want_weights = plain.route(x.double().numpy(), router.double().numpy(), {"top": top, "groups": {"count": count, "keep": keep}})
    assert (chosen.cpu().numpy() == want_chosen).all()
    assert np.abs(weights.cpu().numpy() - want_weights).max() < 1e-5


@pytest.mark.parametrize("path,dtype", [("plain", torch.float32), ("plain", torch.bfloat16), ("stream", torch.float32), ("stream", torch.bfloat16),
                                        ("grouped", torch.bfloat16), (None, torch.bfloat16)])
@pytest.mark.parametrize("tokens,width,ff,experts,top", [(1, 72, 40, 6, 3), (5, 72, 40, 6, 3), (150, 72, 40, 6, 3), (333, 256, 200, 9, 2), (70, 64, 328, 3, 3)])
def test_routed_experts(tokens, width, ff, experts, top, path, dtype):
    """Every way the experts' products are computed: a pair at a time (plain loads, 16-byte loads), and pairs grouped by
    expert on the tensor cores (experts with no pair, with one, with more than a tile of 64)."""
    from lalamo_b200 import ops

    generator = np.random.default_rng(tokens)
    make = lambda *shape: torch.from_numpy(generator.standard_normal(shape)).to(dtype)
    x, gate, up, down = make(tokens, width), make(experts, ff, width) / 8, make(experts, ff, width) / 8, make(experts, width, ff) / 6
    usable = experts - 1 if experts > top else experts   # the last expert gets no pair at all where there are enough others
    chosen = torch.from_numpy(np.stack([generator.permutation(usable)[:top] for _ in range(tokens)]).astype(np.int32))
    weights = torch.from_numpy(generator.random((tokens, top))).float()
    got = ops.moe_experts(x.cuda(), gate.cuda(), up.cuda(), down.cuda(), chosen.cuda(), weights.cuda(), path=path).float().cpu().numpy()
    want = np.zeros((tokens, width))
    for t in range(tokens):
        for e, s in zip(chosen[t].tolist(), weights[t].double().numpy()):
            h = x[t].double().numpy()
            hidden = plain.silu(gate[e].double().numpy() @ h) * (up[e].double().numpy() @ h)
            want[t] += s * (down[e].double().numpy() @ hidden)
    assert np.abs(got - want).max() < (1e-4 if dtype == torch.float32 else 0.06) * np.abs(want).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_of_a_weighted_sum_added_to_the_stream(dtype):
    from lalamo_b200 import ops

    generator = np.random.default_rng(3)
    rows, dim = 37, 200
    make = lambda *shape: torch.from_numpy(generator.standard_normal(shape))
    residual, a, b = make(rows, dim).float(), make(rows, dim).to(dtype), make(rows, dim).to(dtype)
    bias, weight = make(dim).float(), (1 + 0.1 * make(dim)).float()
    y = 0.8 * (a.double() + bias.double()) + 0.9 * b.double()
    want = residual.double() + y / torch.sqrt((y * y).mean(-1, keepdim=True) + 1e-6) * weight.double()
    stream = residual.cuda()
    rounded = torch.empty(rows, dim, dtype=dtype, device="cuda")
    ops.norm_accumulate(stream, ops.ScaledSum([(a.cuda(), 0.8, bias.cuda()), (b.cuda(), 0.9, None)]), weight.cuda(), 1e-6, rounded=rounded)
    assert (stream.cpu().double() - want).abs().max() < 1e-5
    assert torch.equal(rounded.cpu(), stream.cpu().to(dtype))
