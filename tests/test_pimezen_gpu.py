"""The Pimezen design through the framework against the plain implementation of ``plain_pimezen.py``:
each mechanism alone, whole prompts against portions and token-by-token decoding, mixed batches with
pages and state slots that are used again, window and page edges with keys that stand out, long
decoding, several sizes, and greedy generation through the engine's entry point."""

from __future__ import annotations

import json
import math
import random
from pathlib import Path

import pytest
import torch

import plain_pimezen as plain
import schedules
from conftest import note_error

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# Largest |engine - plain| relative to the request's largest |logit|: float32 sums in another order;
# bfloat16 activations rounded between kernels (weights are compared as rounded to bfloat16).
TOLERANCE = {"float32": 1e-5, "bfloat16": 4e-2}  # about twice the worst that any test of this file reaches on a B200 (1.7e-6, 2.0e-2)


def branch(heads, kv_heads, dim, vdim, scale, window, keep_first):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": {"size": window, "keep_first": keep_first}}  # fmt: skip


def layer(left, right, left_scale, right_scale, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}  # fmt: skip


# Three layers that differ from one another in every size: group sizes 2, 1 and 4; value heads narrower
# than, wider than and as wide as key heads; a window shorter than a page, one with no kept tokens, one
# longer than every request; a layer without feed-forward; key widths that are no multiple of four.
CONFIG_P = {
    "architecture": "Pimezen", "vocab": 96, "width": 40, "norm": {"eps": 3e-5},
    "layers": [
        layer(branch(4, 2, 16, 8, 0.3, 12, 3), {"heads": 2, "dim": 8, "vdim": 24, "tau": 4.0, "decay_rank": 4}, 0.6, 1.3,
              {"kind": "dense", "ff": 56, "limit": 1.5}),
        layer(branch(3, 3, 24, 40, 0.21, 7, 0), {"heads": 3, "dim": 18, "vdim": 33, "tau": 9.0, "decay_rank": 3}, 1.2, 0.7, None),
        layer(branch(4, 1, 16, 16, 0.25, 400, 5), {"heads": 1, "dim": 36, "vdim": 96, "tau": 2.5, "decay_rank": 6}, 0.9, 1.0,
              {"kind": "dense", "ff": 24, "limit": 0.7}),
    ],
}  # fmt: skip
# One layer whose window and kept tokens straddle page borders of 16, in a width that the tensor-core products take.
CONFIG_Q = {
    "architecture": "Pimezen", "vocab": 64, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        layer(branch(8, 2, 32, 32, 0.18, 33, 17), {"heads": 4, "dim": 16, "vdim": 32, "tau": 12.0, "decay_rank": 8}, 1.0, 1.0,
              {"kind": "dense", "ff": 128, "limit": 3.0}),
        layer(branch(2, 2, 64, 48, 0.125, 16, 16), {"heads": 2, "dim": 64, "vdim": 16, "tau": 30.0, "decay_rank": 2}, 0.5, 2.0,
              {"kind": "dense", "ff": 72, "limit": 1.0}),
    ],
}  # fmt: skip
# Sizes that no fast path takes: a width that is no multiple of 8 (bfloat16 products on CUDA cores), head widths
# that are no multiples of 8 or of 4 (the scalar attention kernel in bfloat16, in the second layer in float32
# too), one head and one KV head, a feed-forward narrower than the model, a window of one token.
CONFIG_R = {
    "architecture": "Pimezen", "vocab": 51, "width": 36, "norm": {"eps": 1e-4},
    "layers": [
        layer(branch(2, 1, 12, 20, 0.4, 9, 2), {"heads": 3, "dim": 5, "vdim": 7, "tau": 3.0, "decay_rank": 1}, 1.5, 0.5,
              {"kind": "dense", "ff": 17, "limit": 0.9}),
        layer(branch(1, 1, 10, 6, 0.3, 1, 4), {"heads": 2, "dim": 6, "vdim": 10, "tau": 20.0, "decay_rank": 9}, 0.7, 1.4,
              {"kind": "dense", "ff": 64, "limit": 5.0}),
    ],
}  # fmt: skip
CONFIGS = {"P": CONFIG_P, "Q": CONFIG_Q, "R": CONFIG_R}


def random_ids(seed, count, vocab):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from mini_engine_b200.config import PimezenConfig
    from mini_engine_b200.weights import write_random_model

    made = {}
    for name, raw in CONFIGS.items():
        folder = tmp_path_factory.mktemp(f"pimezen_{name}")
        write_random_model(folder, PimezenConfig.from_dict(raw), seed=21, dtype=torch.bfloat16, scale=12.0)
        # As a checkpoint of this design comes: the rank of the decay projection is only a tensor's shape.
        stored = json.loads((folder / "config.json").read_text())
        for entry in stored["layers"]:
            del entry["mixer"]["right"]["decay_rank"]
        (folder / "config.json").write_text(json.dumps(stored))
        made[name] = folder
    return made


def load_plain(folder):
    from safetensors.torch import load_file

    weights = {k: v.to(torch.float32) for k, v in load_file(str(Path(folder) / "model.safetensors")).items()}
    return weights, json.loads((Path(folder) / "config.json").read_text())


def expected_logits(folder, requests):
    weights, config = load_plain(folder)
    return {name: plain.forward_logits(weights, config, toks).float() for name, toks in requests.items()}


def replay(folder, dtype_name, steps, block_size=16, max_tokens=None):
    from mini_engine_b200.engine.replay import Replayer

    replayer = Replayer(folder, DTYPES[dtype_name], max_tokens or schedules.peak_live_tokens(steps), block_size, max_step_tokens=512)
    outputs = {}
    for record in steps:
        logits = replayer.step(record)
        if logits is not None:
            outputs[record["step"]] = logits.clone()
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
    note_error("pimezen " + dtype_name, worst)


LENGTHS = {"P": [70, 45, 133, 9, 97, 33, 1, 2], "Q": [150, 64, 17, 81, 49, 130], "R": [40, 3, 77, 18, 1, 60]}


def requests_for(name):
    return {f"r{i}": random_ids(300 + i, n, CONFIGS[name]["vocab"]) for i, n in enumerate(LENGTHS[name])}


# --------------------------------------------------------------- whole models, every way of cutting


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
@pytest.mark.parametrize("schedule", ["whole", "tail_one_by_one", "changing_portions", "mixed"])
def test_schedules_match_plain(name, dtype_name, schedule, folders):
    """Whole prompts; the last 32 tokens one by one (the windows pass over decoded tokens); portions down
    to two tokens; up to four live requests whose pages and state slots are handed out again."""
    requests = requests_for(name)
    steps = getattr(schedules, schedule)(requests)
    got = replay(folders[name], dtype_name, steps)
    compare(got, expected_logits(folders[name], requests), requests, dtype_name)


@pytest.mark.parametrize("block_size", [4, 16, 32])
def test_float32_does_not_depend_on_the_cut_or_the_batch(folders, block_size):
    """In float32 every kernel's sums for a token depend on that token's position alone, so portions,
    single tokens, mixed batches and other page sizes give the whole prompt's bits."""
    requests = {name: toks for name, toks in list(requests_for("P").items())[:5]}
    whole = replay(folders["P"], "float32", schedules.whole(requests), block_size)
    for maker in (schedules.changing_portions, schedules.mixed, lambda r: schedules.tail_one_by_one(r, 40)):
        cut = replay(folders["P"], "float32", maker(requests), block_size)
        for name, toks in requests.items():
            for position in range(len(toks)):
                assert torch.equal(whole[name][position], cut[name][position]), f"{name} position {position}"


def test_long_decoding_past_every_window(folders):
    """Three prompt tokens, then 200 tokens one by one: the kept first tokens, the windows and the state
    are all that is left of the start."""
    requests = {"long": random_ids(77, 203, CONFIG_Q["vocab"])}
    steps = schedules.tail_one_by_one(requests, tail=200)
    for dtype_name in ("float32", "bfloat16"):
        got = replay(folders["Q"], dtype_name, steps)
        compare(got, expected_logits(folders["Q"], requests), requests, dtype_name)


def test_a_slot_that_is_used_again_starts_from_zero(folders):
    """One state slot and few pages: the second request gets the first one's slot and pages and must
    not see what they held."""
    from mini_engine_b200.engine.replay import Replayer

    a, b = random_ids(5, 40, CONFIG_P["vocab"]), random_ids(6, 37, CONFIG_P["vocab"])
    replayer = Replayer(folders["P"], torch.float32, 64, 16)
    first = replayer.step({"step": 0, "entries": [{"id": "a", "tokens": a, "want": [39]}], "end": ["a"]})
    slot_pages = [list(pool.free_pool) for pool in replayer.manager.pools]
    second = replayer.step({"step": 1, "entries": [{"id": "b", "tokens": b[:20], "want": []}], "end": []})
    assert second is None
    second = replayer.step({"step": 2, "entries": [{"id": "b", "tokens": b[20:], "want": [16]}], "end": ["b"]})
    alone = Replayer(folders["P"], torch.float32, 64, 16).step({"step": 0, "entries": [{"id": "b", "tokens": b, "want": [36]}], "end": ["b"]})
    assert slot_pages and torch.equal(second, alone) and not torch.equal(first, alone)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_the_replay_program_itself(folders, dtype_name, tmp_path):
    """`bin/trace_run` as a process on a model folder of this design: mixed steps in, `done` lines and logit
    files out, equal to the plain implementation."""
    import subprocess
    import sys

    import numpy as np
    from conftest import ROOT

    requests = requests_for("R")
    steps = schedules.mixed(requests)
    out = tmp_path / "out"
    feed = "".join(json.dumps(record) + "\n" for record in steps)
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders["R"]), "--dtype", dtype_name,
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
            outputs[record["step"]] = torch.from_numpy(data.reshape(wanted, CONFIG_R["vocab"]).copy())
    compare(schedules.collect(steps, outputs), expected_logits(folders["R"], requests), requests, dtype_name)


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


def run_attention(q, k, v, r1, r2, talk, scale, window, keep_first, positions, dtype, page_size=16):
    """The kernels of the extended attention on one request whose keys 0..T-1 are cached; queries at `positions`."""
    from mini_engine_b200.csrc import ops

    T, G, D = k.shape
    H, V = q.shape[1], v.shape[2]
    generator = torch.Generator().manual_seed(T)
    k_pages, table = paged(k, page_size, 3 * (-(-T // page_size)), generator)
    generator.manual_seed(T)
    v_pages, _ = paged(v, page_size, 3 * (-(-T // page_size)), generator)
    n = len(positions)
    out = torch.empty(n, H * V, dtype=dtype, device="cuda")
    spread = torch.empty(n, H * G * V, dtype=torch.float32, device="cuda") if talk is not None else None
    cuda = lambda t, dt=None: None if t is None else t.to(device="cuda", dtype=dt or t.dtype).contiguous()  # noqa: E731
    ops.biased_attention(
        q=cuda(q[positions], dtype), k_pages=cuda(k_pages, dtype), v_pages=cuda(v_pages, dtype),
        block_table=cuda(table.view(1, -1)), entry_of_token=torch.zeros(n, dtype=torch.int32, device="cuda"),
        positions=torch.tensor(positions, dtype=torch.int32, device="cuda"), out=out, heads=H, kv_heads=G, head_dim=D,
        value_dim=V, scale=scale, window=window, keep_first=keep_first, r1=cuda(r1, torch.float32),
        r2=cuda(r2, torch.float32), talk=cuda(talk, torch.float32), spread=spread,
    )  # fmt: skip
    torch.cuda.synchronize()
    if talk is not None and window and H // G <= 8 and V <= 256:  # the same through the two-kernel form
        stride = window + keep_first
        again = torch.empty_like(out)
        ops.mixed_attention(
            q=cuda(q[positions], dtype), k_pages=cuda(k_pages, dtype), v_pages=cuda(v_pages, dtype),
            block_table=cuda(table.view(1, -1)), entry_of_token=torch.zeros(n, dtype=torch.int32, device="cuda"),
            positions=torch.tensor(positions, dtype=torch.int32, device="cuda"), out=again, heads=H, kv_heads=G,
            head_dim=D, value_dim=V, scale=scale, window=window, keep_first=keep_first, r1=cuda(r1, torch.float32),
            r2=cuda(r2, torch.float32), talk=cuda(talk, torch.float32),
            scores=torch.full((n * H * stride,), float("nan"), device="cuda"), stats=torch.empty(n * H * 2, device="cuda"),
            stride=stride,
        )  # fmt: skip
        torch.cuda.synchronize()
        tolerance = 3e-5 if dtype == torch.float32 else 3e-2
        assert torch.allclose(again.float(), out.float(), atol=tolerance * max(1.0, float(out.float().abs().max())), rtol=tolerance)
    return out.float().cpu().view(n, H, V)


def plain_attention(q, k, v, r1, r2, talk, scale, window, keep_first):
    H, G = q.shape[1], k.shape[1]
    kv_of_head = torch.arange(H) // (H // G)
    q, k, v = q.double(), k.double(), v.double()
    zero = torch.zeros(H, dtype=torch.float64)
    weights = plain.softmax_weights(q, k[:, kv_of_head], scale, zero if r1 is None else r1.double(),
                                    zero if r2 is None else r2.double(), window if window else 10**9, keep_first)  # fmt: skip
    if talk is not None:
        weights = plain.mix_heads(weights, talk.double())
    return torch.einsum("hij,jhv->ihv", weights, v[:, kv_of_head]).float()


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 16, 8), (6, 3, 40, 72), (3, 1, 8, 33), (2, 2, 128, 128)])
@pytest.mark.parametrize("options", ["all", "no_talk", "no_bias", "plain_window", "no_window"])
def test_attention_options_alone(heads, kv_heads, dim, vdim, options):
    torch.manual_seed(heads * 100 + dim)
    T = 75
    q, k, v = torch.randn(T, heads, dim), torch.randn(T, kv_heads, dim), torch.randn(T, kv_heads, vdim)
    r1 = None if options == "no_bias" else torch.rand(heads) * 2
    r2 = None if options == "no_bias" else torch.rand(heads) + 0.1
    talk = None if options == "no_talk" else torch.randn(heads, heads)
    window = 0 if options == "no_window" else 20
    keep_first = 0 if options in ("plain_window", "no_window") else 6
    want = plain_attention(q, k, v, r1, r2, talk, dim**-0.5, window, keep_first)
    got = run_attention(q, k, v, r1, r2, talk, dim**-0.5, window, keep_first, list(range(T)), torch.float32)
    assert torch.allclose(got, want, atol=3e-5, rtol=1e-4)


@pytest.mark.parametrize("window,keep_first", [(16, 0), (16, 16), (17, 15), (31, 1), (5, 40), (64, 3)])
@pytest.mark.parametrize("offset", ["just_inside", "just_outside", "last_kept", "first_dropped", "far"])
def test_a_key_that_stands_out_at_an_edge(window, keep_first, offset):
    """One key matches one query direction a hundred times better than all others, so that the output is
    that key's value exactly when the mask lets it through: at the window's two sides, at the end of the
    kept tokens, far behind; for the query in a prompt and decoded alone, at page borders."""
    torch.manual_seed(window * 31 + keep_first)
    T, H, G, D, V = 140, 2, 1, 16, 8
    q, k, v = torch.randn(T, H, D) * 0.1, torch.randn(T, G, D) * 0.1, torch.randn(T, G, V)
    position = 131
    key = {"just_inside": position - window + 1, "just_outside": position - window, "last_kept": keep_first - 1,
           "first_dropped": keep_first, "far": 1}[offset]  # fmt: skip
    if key < 0:
        pytest.skip("no kept tokens")
    direction = torch.randn(D)
    q[position] = direction * 3
    k[key, 0] = direction * 3
    r1, r2 = torch.tensor([0.3, 0.0]), torch.tensor([0.5, 1.0])
    want = plain_attention(q, k, v, r1, r2, None, 1.0, window, keep_first)
    seen = position - key < window or key < keep_first
    assert torch.allclose(want[position, 1], v[key, 0], atol=1e-3) == seen  # the test's own premise
    for positions in (list(range(T)), [position]):  # in a prompt of all tokens, and decoded alone
        got = run_attention(q, k, v, r1, r2, None, 1.0, window, keep_first, positions, torch.float32)
        assert torch.allclose(got, want[positions], atol=3e-5, rtol=1e-4)
    talk = torch.tensor([[0.25, 0.75], [-0.5, 1.5]])  # mixed heads: both forms of the kernels at the same edges
    mixed = plain_attention(q, k, v, r1, r2, talk, 1.0, window, keep_first)
    for positions in (list(range(T)), [position]):
        got = run_attention(q, k, v, r1, r2, talk, 1.0, window, keep_first, positions, torch.float32)
        assert torch.allclose(got, mixed[positions], atol=3e-5, rtol=1e-4)
    got = run_attention(q, k, v, r1, r2, None, 1.0, window, keep_first, [position], torch.bfloat16, page_size=8)
    assert torch.allclose(got, want[[position]], atol=3e-2, rtol=3e-2)


# ------------------------------------------------------------- mechanisms alone: linear attention


class FakeContext:
    def __init__(self, counts, slots, fresh):
        cu = [0]
        for n in counts:
            cu.append(cu[-1] + n)
        self.num_entries = len(counts)
        self.cu_tokens = torch.tensor(cu, dtype=torch.int32, device="cuda")
        self.state_slots = torch.tensor(slots, dtype=torch.int32, device="cuda")
        self.fresh = torch.tensor(fresh, dtype=torch.int32, device="cuda")


def scan(proj_parts, columns, a2, bias, state, counts, slots, fresh, heads, dim, vdim, tau):
    from mini_engine_b200.csrc import ops

    tokens = proj_parts.shape[1]
    out = torch.empty(tokens, heads * vdim, dtype=torch.float32, device="cuda")
    prepared = torch.empty(tokens, heads * 3 * dim, dtype=torch.float32, device="cuda")
    ops.gla_scan(proj=proj_parts.cuda().contiguous(), columns=columns, a2t=a2.t().contiguous().cuda(), a2_bias=bias.cuda(),
                 ctx=FakeContext(counts, slots, fresh), state=state, out=out, prepared=prepared, q_scale=dim**-0.5,
                 tau=tau, heads=heads, dim=dim, vdim=vdim)  # fmt: skip
    torch.cuda.synchronize()
    return out.cpu().view(tokens, heads, vdim)


@pytest.mark.parametrize("heads,dim,vdim,rank", [(2, 8, 24, 4), (3, 18, 33, 3), (1, 64, 128, 16), (2, 130, 40, 5)])
def test_recurrence_alone_whole_and_in_portions(heads, dim, vdim, rank):
    """The scan kernel from partial sums (three slices) against the token-by-token recurrence; the same
    sequence in portions of 1, 2, 15, 16 and 17 tokens through a state slot gives the whole's bits; a
    second request beside it, and a slot that held another state, change nothing."""
    torch.manual_seed(dim)
    T, tau = 70, 6.0
    widths = {"q": heads * dim, "k": heads * dim, "v": heads * vdim, "g": heads * vdim, "a": rank}
    columns, width = {}, 0
    for key, w in widths.items():
        columns[key] = width
        width += w
    whole = torch.randn(T, width)
    parts = torch.randn(3, T, width)
    parts[2] = whole - parts[0] - parts[1]
    summed = parts[0] + parts[1] + parts[2]  # what the kernel adds up, in its order
    a2, bias = torch.randn(heads * dim, rank) * 0.5, torch.randn(heads * dim) + 2.0
    col = lambda key, n: summed[:, columns[key] : columns[key] + n].double()  # noqa: E731
    z = col("a", rank) @ a2.double().T + bias.double()
    alpha = torch.sigmoid(z).pow(1 / tau).view(T, heads, dim)
    want, last = plain.recurrence(col("q", heads * dim).view(T, heads, dim) * dim**-0.5, col("k", heads * dim).view(T, heads, dim),
                                  col("v", heads * vdim).view(T, heads, vdim), alpha)  # fmt: skip
    state = torch.full((5, heads, dim, vdim), 7.0, device="cuda")
    got = scan(parts, columns, a2, bias, state, [T], [2], [1], heads, dim, vdim, tau)
    assert torch.allclose(got, want.float(), atol=2e-4, rtol=2e-4)
    assert torch.allclose(state[2].cpu(), last.float(), atol=2e-4, rtol=2e-4)
    assert bool((state[[0, 1, 3, 4]] == 7.0).all())
    # portions, with another request's tokens in front of them in the batch
    other = torch.randn(3, 5, width)
    state2 = torch.full((5, heads, dim, vdim), -3.0, device="cuda")
    done, pieces = 0, []
    for size in (1, 2, 15, 16, 17, T - 51):
        batch = torch.cat((other, parts[:, done : done + size]), dim=1)
        out = scan(batch, columns, a2, bias, state2, [5, size], [4, 1], [1, 1 if done == 0 else 0], heads, dim, vdim, tau)
        pieces.append(out[5:])
        done += size
    assert done == T and torch.equal(torch.cat(pieces), got) and torch.equal(state2[1], state[2])


def test_a_far_token_stays_in_the_state():
    """Decays near one: a large key/value at token 2 still decides the output 300 tokens later, and with
    strong decays it is gone; both as the plain recurrence says."""
    heads, dim, vdim, rank, T = 1, 8, 32, 2, 320
    columns = {"q": 0, "k": dim, "v": 2 * dim, "g": 2 * dim + vdim, "a": 2 * dim + 2 * vdim}
    width = 2 * dim + 2 * vdim + rank
    torch.manual_seed(3)
    proj = torch.randn(1, T, width) * 0.05
    proj[0, 2, dim : 2 * dim] = 4.0
    proj[0, 2, 2 * dim : 2 * dim + vdim] = torch.linspace(-8, 8, vdim)
    proj[0, -1, :dim] = 2.0
    a2 = torch.zeros(dim, rank)
    for bias_value, kept in ((12.0, True), (-2.0, False)):
        bias = torch.full((dim,), bias_value)
        state = torch.zeros(2, heads, dim, vdim, device="cuda")
        got = scan(proj, columns, a2, bias, state, [T], [0], [1], heads, dim, vdim, tau=1.0)
        p = proj[0].double()
        alpha = torch.sigmoid(bias.double()).expand(T, 1, dim)
        want, _ = plain.recurrence(p[:, :dim].view(T, 1, dim) * dim**-0.5, p[:, dim : 2 * dim].view(T, 1, dim),
                                   p[:, 2 * dim : 2 * dim + vdim].view(T, 1, vdim), alpha)  # fmt: skip
        assert torch.allclose(got, want.float(), atol=1e-4, rtol=1e-4)
        assert (float(got[-1].abs().max()) > 10.0) == kept


def test_finish_alone():
    from mini_engine_b200.csrc import ops

    torch.manual_seed(4)
    tokens, heads, vdim = 9, 3, 33
    o = torch.randn(tokens, heads * vdim)
    proj = torch.randn(2, tokens, 200)
    weight = torch.randn(vdim)
    for dtype, tolerance in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        out = torch.empty(tokens, heads * vdim, dtype=dtype, device="cuda")
        ops.gla_finish(o=o.cuda(), proj=proj.cuda(), gate_column=50, weight=weight.cuda(), eps=1e-3, out=out, heads=heads, vdim=vdim)
        gate = (proj[0] + proj[1])[:, 50 : 50 + heads * vdim].double()
        want = plain.unit_rms(o.double().view(tokens, heads, vdim), 1e-3) * weight.double()
        want = want.view(tokens, -1) * torch.nn.functional.silu(gate)
        assert torch.allclose(out.float().cpu(), want.float(), atol=tolerance * 4, rtol=tolerance)


# ------------------------------------------------------------------- mechanisms alone: the small ones


def test_gated_unit_norm_offset_layer_scale_and_branch_sum():
    from mini_engine_b200.csrc import ops

    torch.manual_seed(5)
    tokens, inter, hidden = 7, 20, 24
    both = torch.randn(2, tokens, 2 * inter) * 2
    act = torch.empty(tokens, inter, device="cuda")
    ops.swiglu(both.cuda(), act, 1.702, 1.5, 1.0)
    summed = (both[0] + both[1]).double()
    g, u = summed[:, :inter].clamp(max=1.5), summed[:, inter:].clamp(-1.5, 1.5)
    assert torch.allclose(act.cpu(), (g * torch.sigmoid(1.702 * g) * (u + 1)).float(), atol=1e-5)
    assert float(summed[:, :inter].max()) > 1.5 and float(summed[:, inter:].min()) < -1.5  # the limits did act
    ops.swiglu(both.cuda(), act)  # the defaults are silu(gate) * up
    assert torch.allclose(act.cpu(), (torch.nn.functional.silu(summed[:, :inter]) * summed[:, inter:]).float(), atol=1e-5)

    x, pending, scale, weight = torch.randn(tokens, hidden), torch.randn(3, tokens, hidden), torch.randn(hidden), torch.randn(hidden) * 0.1
    for width in (hidden, hidden - 1):  # the vector path and the scalar one
        xs, out = x[:, :width].contiguous().cuda(), torch.empty(tokens, width, device="cuda")
        ops.add_rmsnorm(xs, pending[:, :, :width].contiguous().cuda(), (weight[:width] + 1.0).cuda(), 1e-4, out, None, scale[:width].contiguous().cuda())
        total = x[:, :width].double() + scale[:width].double() * pending[:, :, :width].double().sum(0)
        assert torch.allclose(xs.cpu(), total.float(), atol=1e-5)
        assert torch.allclose(out.cpu(), plain.zero_centred_norm(total, weight[:width].double(), 1e-4).float(), atol=1e-5)

    a, b = torch.randn(2, tokens, hidden), torch.randn(1, tokens, hidden)
    out = torch.empty(tokens, hidden, device="cuda")
    ops.branch_sum([(a.cuda(), 0.8), (b.cuda(), -1.1)], out)
    assert torch.allclose(out.cpu(), (0.8 * a.double().sum(0) - 1.1 * b[0].double()).float(), atol=1e-5)


def test_one_layer_against_the_plain_layer(folders):
    """The residual stream behind the first layer alone (both mixers, their factors, both layer scales,
    the gated unit), from a model cut down to that layer."""
    from mini_engine_b200.config import PimezenConfig
    from mini_engine_b200.engine.replay import Replayer
    from safetensors.torch import load_file, save_file

    source = folders["P"]
    weights, config = load_plain(source)
    folder = source.parent / (source.name + "_one")
    folder.mkdir(exist_ok=True)
    one = {**config, "layers": config["layers"][:1]}
    (folder / "config.json").write_text(json.dumps(one))
    stored = load_file(str(source / "model.safetensors"))
    save_file({k: v for k, v in stored.items() if not k.startswith(("l1.", "l2."))}, str(folder / "model.safetensors"))
    assert PimezenConfig.from_folder(folder).layers[0].right.decay_rank == 4
    toks = random_ids(9, 50, config["vocab"])
    got = Replayer(folder, torch.float32, 64).step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": list(range(50))}], "end": ["a"]})
    w = {k: v.double() for k, v in weights.items()}
    x = plain.layer(w["embed"][torch.tensor(toks)], w, 0, one["layers"][0], one["norm"]["eps"])
    want = plain.zero_centred_norm(x, w["final.norm"], one["norm"]["eps"]) @ w["embed"].T
    assert torch.allclose(got, want.float(), atol=3e-5 * float(want.abs().max()))


# ------------------------------------------------------------------------ through the entry point


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(folders, dtype_name):
    """`LLMEngine.generate`: the scheduler, portions under a 48-token budget, captured decode steps, state
    slots.  Every generated token is checked teacher-forced: its plain logit lies within the tolerance of
    the largest one at its position."""
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = folders["Q"]
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
        logits = plain.forward_logits(weights, config, (prompt + tokens)[:-1])
        slack = 2 * TOLERANCE[dtype_name] * float(logits.abs().max())
        for i, token in enumerate(tokens):
            row = logits[len(prompt) - 1 + i]
            assert float(row.max() - row[token]) <= slack, f"token {i} of a {len(prompt)}-token prompt"
    again = engine.generate(prompts[:2], SamplingParams(max_tokens=24, ignore_eos=True))
    assert again == got[:2]  # slots and pages of finished requests serve new ones
