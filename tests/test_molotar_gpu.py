"""The Molotar design through the framework against the plain implementation of ``plain_molotar.py``: each
mechanism alone, whole prompts against portions and token-by-token decoding, mixed batches with pages and
state slots that are used again, window edges with keys that stand out, long decoding, several sizes, and
greedy generation through the engine's entry point."""

from __future__ import annotations

import json
import math
import random
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch

import plain_molotar as plain
import schedules
from conftest import note_error

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# Largest |engine - plain| relative to the request's largest |logit|.
TOLERANCE = {"float32": 2e-5, "bfloat16": 5e-2}
# A router's choice that was won by less than this (in score) may fall the other way when activations are rounded
# to bfloat16, and everything behind it follows the other choice.  In bfloat16 the plain implementation is therefore
# told what the engine chose and takes that where its own decision was this close (a differing choice on a clear
# decision fails the test); float32 is compared without any of this.
CLOSE_CALL = 0.02


def attention(heads, kv_heads, dim, vdim, scale, window, rot=None, kv_from=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        out["mask"] = {"size": window}
    if rot:
        out["rot"] = rot
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def routed(ff, limit, experts, top, scale, count, keep):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}  # fmt: skip


ROT_A = {"dims": 8, "base": 500.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 64}}
ROT_B = {"dims": 32, "base": 10000.0, "scaling": {"factor": 16.0, "low": 2.0, "high": 8.0, "original": 300}}
# Five layers that differ from one another: a recurrence first; an attention layer whose keys and values a later layer
# reads with a wider window of its own; value heads wider and narrower than key heads; groups of three, one and two
# heads; a layer without feed-forward; a recurrence with one block and a convolution of one tap (no history); routers
# with groups of two, with one group, and with as many choices as eligible units.
CONFIG_S = {
    "architecture": "Molotar", "vocab": 90, "width": 48, "norm": {"eps": 2e-5}, "postln_alpha": 2.5,
    "embedding": {"scale": 3.0, "bigram": {"buckets": 37, "mul_prev": 11, "mul_cur": 5}},
    "layers": [
        {"type": "rglru", "mixer": {"width": 32, "blocks": 2, "conv": 3}, "mlp": routed(24, 2.0, 6, 2, 1.5, 3, 2)},
        {"type": "attention", "mixer": attention(6, 2, 16, 24, 0.2, 20, ROT_A), "mlp": routed(40, 0.8, 4, 4, 1.0, 1, 1)},
        {"type": "rglru", "mixer": {"width": 64, "blocks": 1, "conv": 1}, "mlp": None},
        {"type": "attention", "mixer": attention(6, 2, 16, 24, 0.35, 33, ROT_A, kv_from=1), "mlp": routed(16, 3.0, 8, 3, 2.5, 4, 3)},
        {"type": "attention", "mixer": attention(2, 2, 24, 8, 0.15, 7, {"dims": 24, "base": 100.0}), "mlp": None},
    ],
}  # fmt: skip
# Widths that the tensor-core products take, windows that straddle pages of 16, an attention layer without a window
# and without rotation whose heads (64 wide, keys and values alike) the tensor-core attention kernels take in bfloat16,
# read again by a later layer with a window; a bigram table of one bucket, alpha 1.
CONFIG_T = {
    "architecture": "Molotar", "vocab": 64, "width": 64, "norm": {"eps": 1e-6}, "postln_alpha": 1.0,
    "embedding": {"scale": 1.0, "bigram": {"buckets": 1, "mul_prev": 1, "mul_cur": 1}},
    "layers": [
        {"type": "attention", "mixer": attention(8, 2, 32, 32, 0.18, 33, ROT_B), "mlp": routed(64, 1.0, 4, 1, 1.0, 2, 1)},
        {"type": "attention", "mixer": attention(2, 1, 64, 64, 0.125, None, None), "mlp": routed(32, 2.0, 8, 2, 2.0, 8, 4)},
        {"type": "rglru", "mixer": {"width": 128, "blocks": 4, "conv": 4}, "mlp": routed(64, 1.5, 2, 2, 0.5, 1, 1)},
        {"type": "attention", "mixer": attention(4, 1, 64, 64, 0.125, 16, None, kv_from=1), "mlp": None},
    ],
}  # fmt: skip
# Sizes that no fast path takes: a width that is no multiple of 8, odd head widths, one head, a window of one token,
# a convolution of five taps, blocks of nine channels, one unit per group.
CONFIG_U = {
    "architecture": "Molotar", "vocab": 51, "width": 36, "norm": {"eps": 1e-4}, "postln_alpha": 4.0,
    "embedding": {"scale": 0.5, "bigram": {"buckets": 101, "mul_prev": 3, "mul_cur": 50}},
    "layers": [
        {"type": "attention", "mixer": attention(1, 1, 10, 6, 0.4, 1, {"dims": 6, "base": 20.0}), "mlp": routed(17, 0.9, 5, 1, 1.0, 5, 3)},
        {"type": "rglru", "mixer": {"width": 27, "blocks": 3, "conv": 5}, "mlp": routed(9, 5.0, 3, 2, 3.0, 1, 1)},
        {"type": "attention", "mixer": attention(3, 1, 14, 20, 0.3, 9, {"dims": 14, "base": 1000.0, "scaling": {"factor": 2.0, "low": 1.0, "high": 3.0, "original": 16}}), "mlp": None},
    ],
}  # fmt: skip
CONFIGS = {"S": CONFIG_S, "T": CONFIG_T, "U": CONFIG_U}
LENGTHS = {"S": [70, 45, 133, 9, 97, 33, 1, 2], "T": [150, 64, 17, 81, 49, 130], "U": [40, 3, 77, 18, 1, 60]}


def random_ids(seed, count, vocab):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from mini_engine_b200.config import MolotarConfig
    from mini_engine_b200.weights import write_random_model

    made = {}
    for name, raw in CONFIGS.items():
        folder = tmp_path_factory.mktemp(f"molotar_{name}")
        write_random_model(folder, MolotarConfig.from_dict(raw), seed=31, dtype=torch.bfloat16, scale=12.0)
        made[name] = folder
    return made


def load_plain(folder):
    from safetensors.torch import load_file

    weights = {k: v.to(torch.float64) for k, v in load_file(str(Path(folder) / "model.safetensors")).items()}
    return weights, json.loads((Path(folder) / "config.json").read_text())


def expected_logits(folder, requests, routing=None):
    """Plain logits per request.  ``routing`` (request -> routed feed-forward -> position -> units) is the engine's
    choice, followed where the plain decision was a close call; few decisions may be that close."""
    weights, config = load_plain(folder)
    out = {}
    for name, toks in requests.items():
        follow = None if routing is None else routing[name]
        out[name] = plain.forward(toks, config, weights, follow=follow, close=CLOSE_CALL)[0].float()
    return out


def replay(folder, dtype_name, steps, block_size=16, max_tokens=None, routing=None, max_live=4, max_step_tokens=512):
    """``routing`` (a dict) is filled with what the routed feed-forwards chose: request -> feed-forward -> position -> units."""
    from mini_engine_b200.engine.replay import Replayer
    from mini_engine_b200.parts import moe as moe_module

    replayer = Replayer(folder, DTYPES[dtype_name], max_tokens or schedules.peak_live_tokens(steps), block_size, max_step_tokens=max_step_tokens, max_live=max_live)
    calls: list = []
    original = moe_module.RoutedExperts.forward

    def recording(self, h, ctx):
        result = original(self, h, ctx)
        calls.append(ctx.buffer("routed.chosen", (h.shape[0], self.top), torch.int32).cpu())
        return result

    if routing is not None:
        moe_module.RoutedExperts.forward = recording
    outputs, held = {}, {}
    try:
        for record in steps:
            calls.clear()
            logits = replayer.step(record)
            if logits is not None:
                outputs[record["step"]] = logits.clone()
            cursor = 0
            for item in record["entries"]:
                start, count = held.get(item["id"], 0), len(item["tokens"])
                for index, chosen in enumerate(calls):
                    per_layer = routing.setdefault(item["id"], {}).setdefault(index, {})
                    for j in range(count):
                        per_layer[start + j] = chosen[cursor + j].tolist()
                cursor, held[item["id"]] = cursor + count, start + count
    finally:
        moe_module.RoutedExperts.forward = original
    replayer.manager.check_invariants([])
    assert all(pool.num_free == pool.num_pages for pool in replayer.manager.pools), "pages were lost"
    assert not replayer.manager.slots.held, "state slots were lost"
    return schedules.collect(steps, outputs)


def compare(got, expected, requests, dtype_name):
    worst = 0.0
    for name, toks in requests.items():
        assert sorted(got[name]) == list(range(len(toks))), f"{name}: positions missing"
        scale = float(expected[name].abs().max())
        for position, row in got[name].items():
            error = float((row - expected[name][position]).abs().max()) / scale
            worst = max(worst, error)
            assert error <= TOLERANCE[dtype_name], f"{name} position {position}: relative error {error:.3g}"
    note_error("molotar " + dtype_name, worst)


def replay_and_compare(folder, dtype_name, steps, requests, **options):
    routing = {} if dtype_name == "bfloat16" else None
    got = replay(folder, dtype_name, steps, routing=routing, **options)
    compare(got, expected_logits(folder, requests, routing), requests, dtype_name)


def requests_for(name):
    return {f"r{i}": random_ids(500 + i, n, CONFIGS[name]["vocab"]) for i, n in enumerate(LENGTHS[name])}


# --------------------------------------------------------------- whole models, every way of cutting


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["S", "T", "U"])
@pytest.mark.parametrize("schedule", ["whole", "tail_one_by_one", "changing_portions", "mixed"])
def test_schedules_match_plain(name, dtype_name, schedule, folders):
    """Whole prompts; the last 32 tokens one by one (the windows pass over decoded tokens); portions down to two
    tokens (shorter than the convolution); up to four live requests whose pages and state slots are handed out again."""
    requests = requests_for(name)
    steps = getattr(schedules, schedule)(requests)
    replay_and_compare(folders[name], dtype_name, steps, requests)


UNUSUAL = {
    # no layer keeps keys and values: no cache group at all, only state slots
    "only_recurrences": [
        {"type": "rglru", "mixer": {"width": 64, "blocks": 2, "conv": 4}, "mlp": routed(32, 2.0, 4, 2, 1.0, 2, 1)},
        {"type": "rglru", "mixer": {"width": 96, "blocks": 3, "conv": 2}, "mlp": None},
    ],
    # the embedding's last token is the only per-request state
    "one_attention": [{"type": "attention", "mixer": attention(2, 2, 32, 32, 0.2, 40, {"dims": 32, "base": 1000.0}), "mlp": routed(32, 2.0, 4, 2, 1.0, 2, 1)}],
    # two readers of one owner that has no window itself: one with a window shorter than a page, one with a long one;
    # 32 units of which a token uses 2 (a decode step reads only the chosen units' weights)
    "readers_of_one_owner": [
        {"type": "attention", "mixer": attention(4, 1, 64, 64, 0.125, None, None), "mlp": None},
        {"type": "attention", "mixer": attention(4, 1, 64, 64, 0.125, 10, None, kv_from=0), "mlp": None},
        {"type": "attention", "mixer": attention(4, 1, 64, 64, 0.3, 200, None, kv_from=0), "mlp": routed(64, 2.0, 32, 2, 1.0, 8, 2)},
    ],
}


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(UNUSUAL))
def test_unusual_layer_combinations(name, dtype_name, tmp_path):
    from mini_engine_b200.config import MolotarConfig
    from mini_engine_b200.weights import write_random_model

    raw = {"architecture": "Molotar", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "postln_alpha": 1.5,
           "embedding": {"scale": 8.0, "bigram": {"buckets": 97, "mul_prev": 5, "mul_cur": 3}}, "layers": UNUSUAL[name]}  # fmt: skip
    write_random_model(tmp_path, MolotarConfig.from_dict(raw), seed=5, dtype=torch.bfloat16, scale=6.0)
    requests = {"a": random_ids(1, 300, 200), "b": random_ids(2, 77, 200), "c": random_ids(3, 1, 200), "d": random_ids(4, 2, 200)}
    for maker in (schedules.whole, schedules.changing_portions, schedules.mixed, lambda r: schedules.tail_one_by_one(r, 32)):
        replay_and_compare(tmp_path, dtype_name, maker(requests), requests)


@pytest.mark.parametrize("block_size", [4, 16, 32])
def test_float32_does_not_depend_on_the_cut_or_the_batch(folders, block_size):
    """In float32 every kernel's sums for a token depend on that token's position alone, so portions, single
    tokens, mixed batches and other page sizes give the whole prompt's bits."""
    requests = {name: toks for name, toks in list(requests_for("S").items())[:5]}
    whole = replay(folders["S"], "float32", schedules.whole(requests), block_size)
    for maker in (schedules.changing_portions, schedules.mixed, lambda r: schedules.tail_one_by_one(r, 40)):
        cut = replay(folders["S"], "float32", maker(requests), block_size)
        for name, toks in requests.items():
            for position in range(len(toks)):
                assert torch.equal(whole[name][position], cut[name][position]), f"{name} position {position}"


def test_long_decoding_past_every_window(folders):
    """Three prompt tokens, then 200 tokens one by one: the windows and the states are all that is left of the start."""
    for name in ("S", "T"):
        requests = {"long": random_ids(77, 203, CONFIGS[name]["vocab"])}
        steps = schedules.tail_one_by_one(requests, tail=200)
        for dtype_name in ("float32", "bfloat16"):
            replay_and_compare(folders[name], dtype_name, steps, requests)


def test_a_slot_that_is_used_again_starts_from_zero(folders):
    """One state slot and few pages: the second request gets the first one's slot (recurrent state, convolution
    history, last token) and pages and must not see what they held."""
    from mini_engine_b200.engine.replay import Replayer

    a, b = random_ids(5, 40, CONFIG_S["vocab"]), random_ids(6, 37, CONFIG_S["vocab"])
    replayer = Replayer(folders["S"], torch.float32, 64, 16, max_live=1)  # one slot: b gets a's
    first = replayer.step({"step": 0, "entries": [{"id": "a", "tokens": a, "want": [39]}], "end": ["a"]})
    second = replayer.step({"step": 1, "entries": [{"id": "b", "tokens": b[:20], "want": []}], "end": []})
    assert second is None
    second = replayer.step({"step": 2, "entries": [{"id": "b", "tokens": b[20:], "want": [16]}], "end": ["b"]})
    alone = Replayer(folders["S"], torch.float32, 64, 16).step({"step": 0, "entries": [{"id": "b", "tokens": b, "want": [36]}], "end": ["b"]})
    assert torch.equal(second, alone) and not torch.equal(first, alone)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_the_replay_program_itself(folders, dtype_name, tmp_path):
    """`bin/trace_run` as a process on a model folder of this design: mixed steps in, `done` lines and logit files out."""
    import subprocess
    import sys

    import numpy as np
    from conftest import ROOT

    requests = requests_for("U")
    steps = schedules.mixed(requests)
    out = tmp_path / "out"
    feed = "".join(json.dumps(record) + "\n" for record in steps)
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders["U"]), "--dtype", dtype_name,
         "--out", str(out), "--max-tokens", str(schedules.peak_live_tokens(steps))],
        input=feed, capture_output=True, text=True, timeout=900,
    )  # fmt: skip
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    outputs = {}
    for record in steps:
        wanted = sum(len(e.get("want", [])) for e in record["entries"])
        if wanted:
            data = np.fromfile(out / f"{record['step']}.f32", dtype="<f4")
            outputs[record["step"]] = torch.from_numpy(data.reshape(wanted, CONFIG_U["vocab"]).copy())
    got = schedules.collect(steps, outputs)
    if dtype_name == "float32":
        compare(got, expected_logits(folders["U"], requests), requests, dtype_name)
    else:  # the process gives the bits of the same steps run in this process (which the schedule tests compare with plain)
        here = replay(folders["U"], dtype_name, steps)
        assert all(torch.equal(got[name][p], here[name][p]) for name, toks in requests.items() for p in range(len(toks)))


def test_the_stream_after_every_layer(folders):
    """The residual stream behind each layer (the normalised sum) against the plain layers, in float32."""
    from mini_engine_b200.engine.replay import Replayer
    from mini_engine_b200.parts import block as block_module

    weights, config = load_plain(folders["S"])
    toks = random_ids(9, 50, config["vocab"])
    _, want = plain.forward(toks, config, weights)
    seen = []
    original = block_module.PostNormBlock.forward

    def recording(self, state, ctx, cache):
        original(self, state, ctx, cache)
        seen.append(state.x.clone())

    block_module.PostNormBlock.forward = recording
    try:
        Replayer(folders["S"], torch.float32, 64).step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": ["a"]})
    finally:
        block_module.PostNormBlock.forward = original
    assert len(seen) == len(config["layers"])
    for index, got in enumerate(seen):
        assert torch.allclose(got.cpu(), want[index].float(), atol=2e-5 * float(want[index].abs().max())), f"layer {index}"


# ---------------------------------------------------------------------- mechanisms alone: attention


def paged(dense, page_size, pages_total, generator):
    """``dense [T, kv, d]`` -> page array ``[pages_total + 1, kv, page_size, d]`` with the request's pages in
    shuffled places and the rest filled with large numbers, and the block table."""
    T, kv, d = dense.shape
    count = -(-T // page_size)
    order = torch.randperm(pages_total, generator=generator)[:count]
    pages = torch.full((pages_total + 1, kv, page_size, d), 1e4, dtype=dense.dtype)
    for t in range(T):
        pages[order[t // page_size], :, t % page_size] = dense[t]
    return pages, order.to(torch.int32)


def run_attention(q, k, v, gate, scale, window, positions, dtype, page_size=16):
    """The attention kernel with a silent participant and gated heads on one request whose keys 0..T-1 are cached."""
    from mini_engine_b200.csrc import ops

    T, G, D = k.shape
    H, V = q.shape[1], v.shape[2]
    generator = torch.Generator().manual_seed(T)
    k_pages, table = paged(k, page_size, 3 * (-(-T // page_size)), generator)
    generator.manual_seed(T)
    v_pages, _ = paged(v, page_size, 3 * (-(-T // page_size)), generator)
    n = len(positions)
    out = torch.empty(n, H * V, dtype=dtype, device="cuda")
    cuda = lambda t, dt=None: None if t is None else t.to(device="cuda", dtype=dt or t.dtype).contiguous()  # noqa: E731
    ops.paged_attention_generic(
        cuda(q[positions].reshape(n, H * D), dtype), cuda(k_pages, dtype), cuda(v_pages, dtype), cuda(table.view(1, -1)),
        torch.zeros(n, dtype=torch.int32, device="cuda"), torch.tensor(positions, dtype=torch.int32, device="cuda"), out,
        H, G, D, scale, window or 0, value_dim=V, sink=True, gate=cuda(None if gate is None else gate[positions], torch.float32),
    )  # fmt: skip
    torch.cuda.synchronize()
    return out.float().cpu().view(n, H, V)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 16, 8), (6, 3, 40, 72), (3, 1, 10, 33), (2, 2, 128, 128)])
@pytest.mark.parametrize("window", [None, 1, 16, 23])
def test_attention_with_a_silent_participant_alone(heads, kv_heads, dim, vdim, window):
    torch.manual_seed(heads * 100 + dim)
    T = 75
    q, k, v = torch.randn(T, heads, dim), torch.randn(T, kv_heads, dim), torch.randn(T, kv_heads, vdim)
    gate = torch.rand(T, heads)
    want = (plain.attend(q.double(), k.double(), v.double(), 0.3, window) * gate.double()[:, :, None]).float()
    got = run_attention(q, k, v, gate, 0.3, window, list(range(T)), torch.float32)
    assert torch.allclose(got, want, atol=2e-5, rtol=2e-5)
    # all scores far below zero: the silent participant takes all the weight and nothing is left for the values
    q_low, k_low = torch.ones(T, heads, dim), torch.full((T, kv_heads, dim), -20.0 * 16 / dim)
    got = run_attention(q_low, k_low, v, None, 0.3, window, list(range(T)), torch.float32)
    assert float(got.abs().max()) < 1e-12
    # all scores far above zero: an ordinary softmax
    k_high = -0.1 * k_low + 0.1 * k
    got = run_attention(q_low, k_high, v, None, 0.3, window, list(range(T)), torch.float32)
    want = plain.attend(q_low.double(), k_high.double(), v.double(), 0.3, window).float()
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("window", [5, 16, 17, 31, 64])
@pytest.mark.parametrize("offset", ["just_inside", "just_outside", "far", "itself"])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_a_key_that_stands_out_at_the_windows_edge(window, offset, dtype_name):
    """One key has a score far above all others and a value that nothing else has: the query's output holds it
    exactly when the key lies inside the window, for a query in a prompt and for one decoded alone, over shuffled
    pages whose free places hold large numbers."""
    torch.manual_seed(window)
    T, H, G, D, V = 150, 4, 2, 16, 24
    query = 140
    target = {"just_inside": query - window + 1, "just_outside": query - window, "far": 3, "itself": query}[offset]
    q, k, v = 0.1 * torch.randn(T, H, D), 0.1 * torch.randn(T, G, D), torch.randn(T, G, V)
    v[:, :, 0] = 0.0
    k[target] = 4.0 * q[query, 0] / q[query, 0].norm()  # aligned with head 0's query
    q[query] = 6.0 * q[query] / q[query].norm(dim=-1, keepdim=True)
    v[target, :, 0] = 100.0
    visible = 0 <= query - target < window
    want = plain.attend(q.double(), k.double(), v.double(), 1.0, window).float()
    dtype = DTYPES[dtype_name]
    if dtype_name == "bfloat16":
        q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
        want = plain.attend(q.double(), k.double(), v.double(), 1.0, window).float()
    for positions in ([query], list(range(query - 20, query + 5))):
        got = run_attention(q, k, v, None, 1.0, window, positions, dtype)
        row = got[positions.index(query)]
        assert (row[0, 0] > 50.0) == visible, f"the marked value is {'missing' if visible else 'seen'}"
        tolerance = 2e-5 if dtype_name == "float32" else 2e-2
        assert torch.allclose(got, want[positions], atol=tolerance * 100.0, rtol=tolerance)


@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("heads,kv_heads,page", [(4, 2, 8), (8, 1, 16), (12, 1, 16), (4, 4, 4)])
@pytest.mark.parametrize("news", [[1, 1, 1, 1], [90, 5, 130, 2], [1, 40, 1, 7]])
@pytest.mark.parametrize("window", [0, 70])
def test_tensor_core_attention_with_a_silent_participant_and_gates(head_dim, heads, kv_heads, page, news, window):
    """The bfloat16 kernels on tensor cores (prompt portions; decode by TMA for groups up to 8 and pages from 8
    tokens, else the tiled one; mixed steps) with the silent participant and the gates, against float64."""
    from test_kernels_gpu import fake_context

    from mini_engine_b200.csrc import attention_bf16, ops

    g = torch.Generator().manual_seed(head_dim + heads + page + len(news) + window)
    lengths = [400, 90, 130, 300]
    total_pages = sum(-(-n // page) for n in lengths) + 3
    order = torch.randperm(total_pages, generator=g).tolist()
    k_pages = torch.randn(total_pages, kv_heads, page, head_dim, generator=g).to(torch.bfloat16)
    v_pages = torch.randn(total_pages, kv_heads, page, head_dim, generator=g).to(torch.bfloat16)
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths) + 1), -1, dtype=torch.int32)
    q_rows, want_rows, gate_rows, entry_of, positions = [], [], [], [], []
    for b, (n, new) in enumerate(zip(lengths, news)):
        q = (0.5 * torch.randn(n, heads, head_dim, generator=g)).to(torch.bfloat16)
        k = torch.randn(n, kv_heads, head_dim, generator=g).to(torch.bfloat16)
        v = torch.randn(n, kv_heads, head_dim, generator=g).to(torch.bfloat16)
        if b % 2:
            q = -q.abs()  # scores mostly far below zero: the silent participant holds most of the weight
            k = k.abs()
        gate = torch.rand(n, heads, generator=g)
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
        for p in range(n):
            k_pages[table[b, p // page], :, p % page] = k[p]
            v_pages[table[b, p // page], :, p % page] = v[p]
        want = plain.attend(q.double(), k.double(), v.double(), head_dim**-0.5, window or None) * gate.double()[:, :, None]
        q_rows.append(q[n - new :]), want_rows.append(want[n - new :]), gate_rows.append(gate[n - new :])
        entry_of += [b] * new
        positions += list(range(n - new, n))
    data = dict(new_counts=news, lengths=lengths, entry_of=torch.tensor(entry_of, dtype=torch.int32).cuda(),
                positions=torch.tensor(positions, dtype=torch.int32).cuda())  # fmt: skip
    q_all = torch.cat(q_rows).reshape(-1, heads * head_dim).contiguous().cuda()
    want = torch.cat(want_rows).reshape(-1, heads * head_dim).float()
    out = torch.full_like(q_all, float("nan"))
    assert attention_bf16.supports(head_dim, heads, kv_heads)
    ops.paged_attention(
        q=q_all, k_pages=k_pages.cuda(), v_pages=v_pages.cuda(), block_table=table.cuda(), ctx=fake_context(data), out=out,
        heads=heads, kv_heads=kv_heads, head_dim=head_dim, scale=head_dim**-0.5, window=window, sink=True,
        gate=torch.cat(gate_rows).contiguous().cuda(),
    )  # fmt: skip
    torch.cuda.synchronize()
    assert attention_bf16.take_error() == 0
    error = float((out.float().cpu() - want).abs().max()) / float(want.abs().max())
    assert error < 1.5e-2, error


def test_norm_over_whole_projections_rotation_gates_and_cache_write():
    """q over all its heads at once, k over all of its, rotation of the first part of every head with stretched
    frequencies, v untouched, sigmoid gates, the write into shuffled slots."""
    from mini_engine_b200.csrc import ops
    from mini_engine_b200.parts.rotary import RotaryEncoding

    torch.manual_seed(3)
    T, H, G, D, V, page = 21, 3, 2, 12, 20, 4
    rot = {"dims": 8, "base": 50.0, "scaling": {"factor": 3.0, "low": 1.0, "high": 2.0, "original": 16}}
    width = (H + G) * D + G * V + H
    parts = torch.randn(3, T, width)  # three partial sums
    whole = parts.sum(0).double()
    qw, kw = 1 + 0.1 * torch.randn(H * D), 1 + 0.1 * torch.randn(G * D)
    positions = torch.arange(100, 100 + T, dtype=torch.int32)
    slots = torch.randperm(8 * page)[:T].to(torch.int32)
    encoding = RotaryEncoding("", 0, head_dim=D, theta=rot["base"], rotary_dim=rot["dims"], wavelength_scaling=rot["scaling"])
    angles = torch.empty(T, rot["dims"] // 2, 2, device="cuda")
    ops.rope_table(encoding.inv_freq().cuda(), positions.cuda(), angles)
    q_out = torch.empty(T, H * D, device="cuda")
    k_pages, v_pages = torch.zeros(9, G, page, D, device="cuda"), torch.zeros(9, G, page, V, device="cuda")
    gates = torch.empty(T, H, device="cuda")
    ops.qk_wide_norm_rope_store(
        qkv=parts.cuda(), heads=H, kv_heads=G, head_dim=D, value_dim=V, q_weight=qw.cuda(), k_weight=kw.cuda(), eps=1e-3,
        cos_sin=angles, q_out=q_out, page_size=page, slot_mapping=slots.cuda(), k_pages=k_pages, v_pages=v_pages, gates=H,
        gate_out=gates,
    )  # fmt: skip
    torch.cuda.synchronize()
    place = list(range(100, 100 + T))
    want_q = plain.rotate(plain.rms_norm(whole[:, : H * D], qw, 1e-3).view(T, H, D), place, rot).float()
    want_k = plain.rotate(plain.rms_norm(whole[:, H * D : (H + G) * D], kw, 1e-3).view(T, G, D), place, rot).float()
    want_v = whole[:, (H + G) * D : (H + G) * D + G * V].view(T, G, V).float()
    assert torch.allclose(q_out.cpu().view(T, H, D), want_q, atol=1e-5, rtol=1e-5)
    got_k = torch.stack([k_pages[int(s) // page, :, int(s) % page] for s in slots]).cpu()
    got_v = torch.stack([v_pages[int(s) // page, :, int(s) % page] for s in slots]).cpu()
    assert torch.allclose(got_k, want_k, atol=1e-5, rtol=1e-5) and torch.allclose(got_v, want_v, atol=1e-6)
    assert torch.allclose(gates.cpu(), torch.sigmoid(whole[:, -H:]).float(), atol=1e-6)


# ------------------------------------------------------------------ mechanisms alone: the recurrence


def recurrence_weights(C, B, K, hidden, seed, lam=None):
    g = torch.Generator().manual_seed(seed)
    n = lambda *shape, s=1.0: s * torch.randn(*shape, generator=g)  # noqa: E731
    return {"y": n(C, hidden, s=0.3), "y.b": n(C, s=0.2), "x": n(C, hidden, s=0.3), "x.b": n(C, s=0.2), "conv": n(C, K, s=0.5),
            "conv.b": n(C, s=0.1), "ra": n(B, C // B, C // B, s=0.4), "ra.b": n(B, C // B, s=0.3), "ri": n(B, C // B, C // B, s=0.4),
            "ri.b": n(B, C // B, s=0.3), "lam": n(C, s=1.0) if lam is None else torch.full((C,), lam), "o": torch.eye(C)}  # fmt: skip


def run_recurrence(h, w, B, entries, state, splits=2):
    """The two kernels over a flat batch: ``entries`` are (first token, count, slot, fresh)."""
    from mini_engine_b200.csrc import ops

    T = h.shape[0]
    C, K = w["conv"].shape
    whole = torch.cat((h @ w["y"].T, h @ w["x"].T), dim=1)
    noise = torch.randn(splits - 1, T, 2 * C)
    proj = torch.cat((noise, (whole - noise.sum(0)).unsqueeze(0))).cuda().contiguous()  # partial sums that add up
    entry_of_token = torch.zeros(T, dtype=torch.int32)
    cu = [0]
    for index, (_first, count, _slot, _fresh) in enumerate(entries):
        entry_of_token[cu[-1] : cu[-1] + count] = index
        cu.append(cu[-1] + count)
    assert cu[-1] == T
    ctx = SimpleNamespace(
        entry_of_token=entry_of_token.cuda(), cu_tokens=torch.tensor(cu, dtype=torch.int32).cuda(),
        state_slots=torch.tensor([e[2] for e in entries], dtype=torch.int32).cuda(),
        fresh=torch.tensor([int(e[3]) for e in entries], dtype=torch.int32).cuda(), num_entries=len(entries),
    )  # fmt: skip
    out = torch.empty(T, C, device="cuda")
    f = lambda t: t.float().cuda().contiguous()  # noqa: E731
    ops.rglru(
        proj=proj, in_bias=f(torch.cat((w["y.b"], w["x.b"]))), taps=f(w["conv"]), conv_bias=f(w["conv.b"]),
        ra_t=f(w["ra"].transpose(1, 2)), ra_bias=f(w["ra.b"].reshape(-1)), ri_t=f(w["ri"].transpose(1, 2)),
        ri_bias=f(w["ri.b"].reshape(-1)), lam=f(w["lam"]), ctx=ctx, state=state, decay=torch.empty(T, C, device="cuda"),
        driven=torch.empty(T, C, device="cuda"), conv=torch.empty(T, C, device="cuda"), out=out, sharpness=8.0,
    )  # fmt: skip
    torch.cuda.synchronize()
    return out.cpu()


@pytest.mark.parametrize("C,B,K", [(32, 2, 3), (64, 1, 1), (27, 3, 5), (256, 2, 4), (48, 48, 2)])
def test_recurrence_alone_whole_and_in_portions(C, B, K):
    """The whole sequence in one entry against the plain recurrence; then in portions of 1, 2, 3 and more tokens
    (shorter than the convolution) through a state slot, beside another request, bit for bit the same."""
    torch.manual_seed(C + K)
    T, hidden = 61, 24
    w = recurrence_weights(C, B, K, hidden, seed=C)
    h = torch.randn(T, hidden)
    m = {"width": C, "blocks": B}
    want = plain.rglru(h.double(), m, {"p." + k: v.double() for k, v in w.items()}, "p.").float()
    state = torch.full((4, K, C), 7.0, device="cuda")  # what an earlier request left in the slots
    whole = run_recurrence(h, w, B, [(0, T, 2, True)], state)
    assert torch.allclose(whole, want, atol=2e-5, rtol=2e-5)
    other = torch.randn(30, hidden)
    other_whole = run_recurrence(other, w, B, [(0, 30, 0, True)], state)
    state.fill_(-3.0)
    done, other_done, pieces, other_pieces = 0, 0, [], []
    for size in (1, 2, 1, 3, 2, 17, 1, 1, 5, 28):
        other_size = min(3, 30 - other_done)
        batch = [h[done : done + size]] + ([other[other_done : other_done + other_size]] if other_size else [])
        entries = [(done, size, 1, done == 0)] + ([(other_done, other_size, 3, other_done == 0)] if other_size else [])
        out = run_recurrence(torch.cat(batch), w, B, entries, state, splits=3)
        pieces.append(out[:size]), other_pieces.append(out[size:])
        done, other_done = done + size, other_done + other_size
    assert done == T and other_done == 30
    # not bit for bit here: this test cuts the projections into other random partial sums for every call
    assert torch.allclose(torch.cat(pieces), whole, atol=2e-5, rtol=2e-5)
    assert torch.allclose(torch.cat(other_pieces), other_whole, atol=2e-5, rtol=2e-5)


def test_a_far_token_stays_in_the_state_or_is_gone():
    """With decays close to one a token 300 steps back still shows in the output; with fast decays it is gone."""
    torch.manual_seed(1)
    C, B, K, hidden, T = 16, 1, 2, 8, 301
    h = 0.01 * torch.randn(T, hidden)
    h[0] = 5.0 * torch.randn(hidden)
    base = h.clone()
    base[0] = 0.01 * torch.randn(hidden)
    for lam, stays in ((-9.0, True), (1.0, False)):
        w = recurrence_weights(C, B, K, hidden, seed=2, lam=lam)
        m = {"width": C, "blocks": B}
        plain_w = {"p." + k: v.double() for k, v in w.items()}
        want, want_base = plain.rglru(h.double(), m, plain_w, "p.").float(), plain.rglru(base.double(), m, plain_w, "p.").float()
        state = torch.zeros(2, K, C, device="cuda")
        run_recurrence(h[:200], w, B, [(0, 200, 0, True)], state)
        got = torch.cat([run_recurrence(h[t : t + 1], w, B, [(t, 1, 0, False)], state, splits=1) for t in range(200, T)])
        assert torch.allclose(got, want[200:], atol=1e-5, rtol=1e-4)
        differs = float((want[-1] - want_base[-1]).abs().max())
        assert (differs > 1e-3) == stays


# -------------------------------------------------------------- mechanisms alone: router, units, ends


@pytest.mark.parametrize("experts,top,count,keep", [(8, 3, 4, 3), (6, 2, 3, 2), (4, 4, 1, 1), (5, 1, 5, 3), (16, 4, 2, 1), (3, 2, 1, 1)])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_router_alone(experts, top, count, keep, dtype_name):
    from mini_engine_b200.csrc import ops

    torch.manual_seed(experts * 10 + top)
    T, hidden = 40, 24
    h = torch.randn(T, hidden).to(DTYPES[dtype_name])
    weight = torch.randn(experts, hidden)
    router = {"experts": experts, "top": top, "scale": 1.7, "groups": {"count": count, "keep": keep}}
    chosen, weights, _ = plain.route(h.double(), router, weight.double())
    dense = torch.empty(T, experts, device="cuda")
    ids = torch.empty(T, top, dtype=torch.int32, device="cuda")
    picked = torch.empty(T, top, device="cuda")
    ops.route(h=h.cuda(), router=weight.cuda(), weights=dense, chosen=ids, chosen_weight=picked, top=top, group_count=count,
              group_keep=keep, weight_scale=1.7)  # fmt: skip
    torch.cuda.synchronize()
    for t in range(T):
        assert ids[t].tolist() == chosen[t], f"token {t}"
        assert torch.allclose(picked[t].cpu(), torch.tensor(weights[t]), atol=1e-5)
        want = torch.zeros(experts)
        want[torch.tensor(chosen[t])] = torch.tensor(weights[t])
        assert torch.allclose(dense[t].cpu(), want, atol=1e-5)
        assert math.isclose(float(dense[t].sum()), 1.7, rel_tol=1e-5)


@pytest.mark.parametrize("tokens,top,units,hidden,inter", [(300, 2, 8, 64, 96), (257, 3, 5, 128, 40), (1000, 1, 3, 72, 264)])
def test_rows_sorted_by_unit_and_grouped_products_alone(tokens, top, units, hidden, inter):
    """Every (token, choice) gets one row in its unit's padded run; the grouped products read the weights of a run's
    unit; a token's rows come back together with its weights in the order of its choices."""
    from mini_engine_b200.csrc import ops

    g = torch.Generator().manual_seed(tokens + units)
    pad = ops.GROUP_PAD
    chosen = torch.stack([torch.randperm(units, generator=g)[:top] for _ in range(tokens)]).to(torch.int32)
    chosen[: tokens // 3] = chosen[0]  # one unit with many more rows than the others, one maybe with none
    weight = torch.rand(tokens, top, generator=g)
    capacity = -(-(tokens * top + units * (pad - 1)) // pad) * pad
    row_of = torch.empty(tokens, top, dtype=torch.int32, device="cuda")
    token_of = torch.empty(capacity, dtype=torch.int32, device="cuda")
    unit_of_block = torch.empty(capacity // pad, dtype=torch.int32, device="cuda")
    ops.sort_by_unit(chosen=chosen.cuda(), units=units, pad=pad, row_of=row_of, token_of=token_of, unit_of_block=unit_of_block)
    torch.cuda.synchronize()
    rows, owner, blocks = row_of.cpu(), token_of.cpu(), unit_of_block.cpu()
    assert len(set(rows.flatten().tolist())) == tokens * top and int(rows.min()) >= 0 and int(rows.max()) < capacity
    for t in range(tokens):
        for k in range(top):
            row = int(rows[t, k])
            assert int(owner[row]) == t and int(blocks[row // pad]) == int(chosen[t, k])
    assert int((owner >= 0).sum()) == tokens * top
    h = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    gathered = torch.empty(capacity, hidden, dtype=torch.bfloat16, device="cuda")
    ops.gather_rows(h.cuda(), token_of, gathered)
    w_gate_up = (0.2 * torch.randn(units, 2 * inter, hidden, generator=g)).to(torch.bfloat16)
    w_down = (0.2 * torch.randn(units, hidden, inter, generator=g)).to(torch.bfloat16)
    act = torch.empty(capacity, inter, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tensor_core_grouped(ops.GemmPlan(w_gate_up.reshape(-1, hidden).contiguous().cuda()), gathered, act, unit_of_block,
                                 2 * inter, inter, dual_rows=inter, slope=1.702, limit=1.5, offset=1.0)  # fmt: skip
    down = torch.empty(capacity, hidden, dtype=torch.float32, device="cuda")
    ops.gemm_tensor_core_grouped(ops.GemmPlan(w_down.reshape(-1, inter).contiguous().cuda()), act, down, unit_of_block, hidden, hidden)
    out = torch.empty(tokens, hidden, device="cuda")
    ops.combine_rows(down, row_of, weight.cuda(), out)
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    want = torch.zeros(tokens, hidden, dtype=torch.float64)
    for t in range(tokens):
        for k in range(top):
            u = int(chosen[t, k])
            both = w_gate_up[u].double() @ h[t].double()
            gate, up = both[:inter].clamp(max=1.5), both[inter:].clamp(-1.5, 1.5)
            unit_act = (gate * torch.sigmoid(1.702 * gate) * (up + 1.0)).to(torch.bfloat16).double()
            assert torch.allclose(act[int(rows[t, k])].double().cpu(), unit_act, atol=2e-2, rtol=2e-2)
            want[t] += float(weight[t, k]) * (w_down[u].double() @ unit_act)
    assert torch.allclose(out.cpu().double(), want, atol=2e-2 * float(want.abs().max()), rtol=2e-2)


def test_a_long_prompt_takes_the_sorted_form_and_matches_plain(folders):
    """A bfloat16 prompt of 300 tokens in one step (rows sorted by unit), the same prompt in portions of at most 64
    tokens (all units, masked), and the plain implementation."""
    requests = {"long": random_ids(91, 300, CONFIG_T["vocab"])}
    replay_and_compare(folders["T"], "bfloat16", schedules.whole(requests), requests)
    replay_and_compare(folders["T"], "bfloat16", schedules.changing_portions(requests), requests)


def test_sum_scaled_stream_norm_written_back():
    """``x = w * rms_norm(alpha * x + sum of the partial sums)`` in place, and the same rounded for the next sublayer."""
    from mini_engine_b200.csrc import ops

    torch.manual_seed(0)
    for hidden in (48, 36, 1024):
        x, parts, w = torch.randn(9, hidden), torch.randn(3, 9, hidden), 1 + 0.1 * torch.randn(hidden)
        want = plain.rms_norm(2.5 * x.double() + parts.double().sum(0), w.double(), 1e-5).float()
        xd, out = x.cuda(), torch.empty(9, hidden, dtype=torch.bfloat16, device="cuda")
        ops.add_rmsnorm(xd, parts.cuda(), w.cuda(), 1e-5, out, None, None, 2.5, True)
        torch.cuda.synchronize()
        assert torch.allclose(xd.cpu(), want, atol=1e-5, rtol=1e-5) and torch.equal(out.cpu(), xd.cpu().to(torch.bfloat16))


def test_pair_embedding_first_tokens_and_the_token_carried_between_steps():
    from mini_engine_b200.csrc import ops

    torch.manual_seed(0)
    vocab, hidden, buckets = 30, 20, 7
    table, pairs = torch.randn(vocab, hidden), torch.randn(buckets + 1, hidden)
    cfg = {"embedding": {"scale": 1.5, "bigram": {"buckets": buckets, "mul_prev": 13, "mul_cur": 3}}}
    a, b = random_ids(1, 12, vocab), random_ids(2, 9, vocab)
    want_a = plain.embed(a, cfg, {"embed": table, "bigram": pairs}, torch.float32)
    want_b = plain.embed(b, cfg, {"embed": table, "bigram": pairs}, torch.float32)
    last = torch.full((4,), 29, dtype=torch.int32, device="cuda")  # what other requests left behind

    def step(entries):
        ids = [t for toks, _slot, _fresh in entries for t in toks]
        cu = [0]
        for toks, _, _ in entries:
            cu.append(cu[-1] + len(toks))
        ctx = SimpleNamespace(
            token_ids=torch.tensor(ids, dtype=torch.int32).cuda(),
            entry_of_token=torch.tensor([i for i, e in enumerate(entries) for _ in e[0]], dtype=torch.int32).cuda(),
            cu_tokens=torch.tensor(cu, dtype=torch.int32).cuda(), state_slots=torch.tensor([e[1] for e in entries], dtype=torch.int32).cuda(),
            fresh=torch.tensor([int(e[2]) for e in entries], dtype=torch.int32).cuda(),
        )  # fmt: skip
        out = torch.empty(len(ids), hidden, device="cuda")
        rounded = torch.empty(len(ids), hidden, dtype=torch.bfloat16, device="cuda")
        ops.pair_embedding(table=table.cuda(), pair_table=pairs.cuda(), ctx=ctx, last_token=last, out=out, rounded=rounded,
                           multiplier=1.5, buckets=buckets, mul_prev=13, mul_cur=3)  # fmt: skip
        torch.cuda.synchronize()
        assert torch.equal(rounded.cpu(), out.cpu().to(torch.bfloat16))
        return out.cpu()

    first = step([(a[:5], 2, True), (b[:1], 0, True)])
    second = step([(a[5:6], 2, False), (b[1:8], 0, False)])
    third = step([(b[8:], 0, False), (a[6:], 2, False)])
    got_a = torch.cat((first[:5], second[:1], third[1:]))
    got_b = torch.cat((first[5:], second[1:], third[:1]))
    assert torch.allclose(got_a, want_a, atol=1e-6) and torch.allclose(got_b, want_b, atol=1e-6)
    assert last.tolist() == [b[-1], 29, a[-1], 29]


# ------------------------------------------------------------------------ through the entry point


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["S", "T"])
def test_greedy_generation_through_the_engine(folders, dtype_name, name):
    """`LLMEngine.generate`: the scheduler, portions under a 48-token budget, captured decode steps, state slots.
    Every generated token is checked teacher-forced: its plain logit lies within the tolerance of the largest one
    at its position."""
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = folders[name]
    weights, config = load_plain(folder)
    prompts = [random_ids(40 + i, n, config["vocab"]) for i, n in enumerate((19, 70, 3, 41, 100))]
    engine = LLMEngine.from_pretrained(
        folder, EngineConfig(block_size=16, num_blocks=64, max_model_len=256, max_num_seqs=3, max_num_batched_tokens=48,
                             dtype=DTYPES[dtype_name])  # fmt: skip
    )
    got = engine.generate(prompts, SamplingParams(max_tokens=24, ignore_eos=True))
    assert engine.stats.graph_steps > 0
    for prompt, tokens in zip(prompts, got):
        assert len(tokens) == 24
        gaps: list = []
        logits = plain.forward((prompt + tokens)[:-1], config, weights, gaps=gaps)[0].float()
        slack = 2 * TOLERANCE[dtype_name] * float(logits.abs().max())
        for i, token in enumerate(tokens):
            if dtype_name == "bfloat16" and any(min(layer[: len(prompt) + i]) < CLOSE_CALL / 4 for layer in gaps):
                break  # a routing decision that rounding may turn: what follows is another sequence's business
            row = logits[len(prompt) - 1 + i]
            assert float(row.max() - row[token]) <= slack, f"token {i} of a {len(prompt)}-token prompt"
    again = engine.generate(prompts[:2], SamplingParams(max_tokens=24, ignore_eos=True))
    assert again == got[:2]  # slots and pages of finished requests serve new ones


def test_the_command_line_and_sampling_with_temperature(folders, capsys):
    """`python -m mini_engine_b200.cli.generate` on a folder of this design: greedy output equals the engine's, and a
    run with temperature draws tokens of the vocabulary through the device sampler."""
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.cli import generate

    folder = str(folders["S"])
    prompts = [random_ids(70 + i, n, CONFIG_S["vocab"]) for i, n in enumerate((12, 30))]
    ids = ";".join(",".join(map(str, p)) for p in prompts)
    common = ["--model", folder, "--dtype", "fp32", "--max-tokens", "6", "--ignore-eos", "--num-blocks", "32", "--max-model-len", "128",
              "--max-num-seqs", "2", "--prompt-ids", ids]  # fmt: skip
    assert generate.main(common) == 0
    greedy = capsys.readouterr().out
    engine = LLMEngine.from_pretrained(folder, EngineConfig(block_size=16, num_blocks=32, max_model_len=128, max_num_seqs=2, dtype=torch.float32))
    want = engine.generate(prompts[:1], SamplingParams(max_tokens=6, ignore_eos=True)) + engine.generate(prompts[1:], SamplingParams(max_tokens=6, ignore_eos=True))
    for prompt, tokens in zip(prompts, want):
        assert f"prompt ({len(prompt)} tokens) -> {tokens}" in greedy
    assert generate.main(common + ["--temperature", "0.8", "--seed", "3"]) == 0
    drawn = capsys.readouterr().out.splitlines()[:2]
    for line, prompt in zip(drawn, prompts):
        tokens = json.loads(line.split("-> ")[1])
        assert line.startswith(f"prompt ({len(prompt)} tokens)") and len(tokens) == 6 and all(0 <= t < CONFIG_S["vocab"] for t in tokens)


def test_preempted_requests_start_again_from_zero_state(folders):
    """A pool so small that running requests are preempted: their pages and state slots go back, they are computed
    again from their first token (the recurrent state, the convolution's history and the last token start from
    nothing), and the tokens are those of a run with room for everyone."""
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = folders["S"]
    prompts = [random_ids(90 + i, n, CONFIG_S["vocab"]) for i, n in enumerate((40, 33, 25, 47))]
    params = SamplingParams(max_tokens=30, ignore_eos=True)
    roomy = LLMEngine.from_pretrained(folder, EngineConfig(block_size=16, num_blocks=64, max_model_len=128, max_num_seqs=4, dtype=torch.float32))
    want = roomy.generate(prompts, params)
    tight = LLMEngine.from_pretrained(folder, EngineConfig(block_size=16, num_blocks=11, max_model_len=128, max_num_seqs=4, dtype=torch.float32))
    got = tight.generate(prompts, params)
    assert tight.scheduler.num_preemptions > 0
    assert got == want
