"""The Tikizen design in the engine against its plain statement: every kernel alone, whole prompts, every way of
cutting a request into steps, batches, slots and pages used again, long decoding, keys at the edges of chunks, and
greedy generation through the engine's own entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_tikizen as pt
from helpers import cut, random_tokens, rel_err
from tikizen_cases import CASE_P, CASE_Q, CASE_R, CASES, for_dtype, make_weights

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
SEEDS = {"P": 11, "Q": 12, "R": 13, "S": 14}


def assert_close(got, want, dtype):
    """float32: every row within 2e-4 of its largest value.  bfloat16: the rows are judged together, by their median
    error and the nineteenth of twenty (a routed feed-forward may choose another expert where two logits are closer
    than bfloat16 tells apart, and a head that is nearly zero before it is brought to unit size amplifies rounding)."""
    if dtype == torch.float32:
        assert rel_err(got, want) < TOL[dtype]
        return
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape and bool(torch.isfinite(got).all())
    err = (got - want).abs().amax(dim=1) / want.abs().amax(dim=1).clamp_min(1e-30)
    assert float(err.median()) < 2.5e-2, float(err.median())
    assert float(torch.quantile(err, 0.95)) < TOL[dtype], float(torch.quantile(err, 0.95))


def on_device(w, dtype):
    return {k: v.to(dtype).cuda() for k, v in w.items()}


def make_runner(case, w, dtype, n_pages=24, max_requests=3, page_size=16, use_graphs=False):
    from inferrs_b200.engine.loading import spec_from_config
    from inferrs_b200.engine.runner import ModelRunner
    from inferrs_b200.runtime import Runtime
    spec, _ = spec_from_config(case, tensor_shapes={k: tuple(v.shape) for k, v in w.items()})
    rt = Runtime.cuda(dtype)
    return ModelRunner(spec, on_device(w, dtype), rt, page_size=page_size, n_pages=n_pages, max_requests=max_requests,
                       use_graphs=use_graphs)


def entry(rid, tokens, want=None):
    from inferrs_b200.engine.batch import StepEntry
    return StepEntry(rid, tokens, list(range(len(tokens))) if want is None else want)


def dev(v, dtype=torch.int32):
    return torch.tensor(v, dtype=dtype, device="cuda")


def act(x, dtype):
    return x.to(dtype).cuda().contiguous()


# ---------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_whole_prompt_and_every_cutting_match_the_plain_statement(name, dtype):
    case, w = for_dtype(CASES[name], dtype), make_weights(CASES[name], SEEDS[name])
    toks = random_tokens(131, case["vocab"], seed=3)       # past chunk edges at 40, 48, 56, 80, 96, 112, 120
    want = pt.forward(case, w, toks)
    runner = make_runner(case, w, dtype)
    runner.admit("whole")
    got = runner.step([entry("whole", toks)])
    assert_close(got, want, dtype)
    runner.release("whole")
    # one token a step from an empty cache: the first tokens of a sequence, and decoding through cache and state
    runner.admit("single")
    rows = [runner.step([entry("single", [t])]) for t in toks[:60]]
    assert_close(torch.cat(rows), want[:60], dtype)
    runner.release("single")
    # portions of changing size, down to two tokens and one, another request's portions beside them
    other = random_tokens(50, case["vocab"], seed=4)
    want_other = pt.forward(case, w, other)
    runner.admit("cut")
    runner.admit("other")
    at, o_at, rows, o_rows = 0, 0, [], []
    for n in cut(len(toks), [7, 2, 30, 1, 1, 2, 17, 3, 41]):
        entries = [entry("cut", toks[at:at + n])]
        if o_at < len(other):
            entries.insert(o_at % 2, entry("other", other[o_at:o_at + 6]))
        out = runner.step(entries)
        k = 0
        for e in entries:
            (rows if e.rid == "cut" else o_rows).append(out[k:k + len(e.tokens)])
            k += len(e.tokens)
        o_at += 6
        at += n
    assert_close(torch.cat(rows), want, dtype)
    assert_close(torch.cat(o_rows), want_other[:sum(r.shape[0] for r in o_rows)], dtype)
    runner.manager.check_invariants()


def test_a_second_norm_without_a_feed_forward():
    case, w = CASE_Q, make_weights(CASE_Q, 17, bare_norm2=True)
    assert "l2.norm2" in w
    toks = random_tokens(40, case["vocab"], seed=5)
    runner = make_runner(case, w, torch.float32)
    runner.admit(0)
    assert rel_err(runner.step([entry(0, toks)]), pt.forward(case, w, toks)) < TOL[torch.float32]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_unequal_requests_in_one_batch_slots_and_pages_used_again(name, dtype):
    """Two state slots and pages for two requests; five requests of unequal length take turns, decoding side by side
    with portions of the next ones.  Every request must give what it gives alone (the plain statement knows no
    batches, slots or pages)."""
    case, w = for_dtype(CASES[name], dtype), make_weights(CASES[name], SEEDS[name])
    lens = {"a": 50, "b": 23, "c": 64, "d": 9, "e": 37}
    toks = {k: random_tokens(n, case["vocab"], seed=ord(k)) for k, n in lens.items()}
    want = {k: pt.forward(case, w, t) for k, t in toks.items()}
    runner = make_runner(case, w, dtype, n_pages=9, max_requests=2)      # 144 cached tokens: no three requests fit
    got = {k: [] for k in lens}
    at = {k: 0 for k in lens}
    live, waiting = [], list(lens)
    sizes = [13, 1, 1, 2, 5, 1, 30, 1]
    i = 0
    while live or waiting:
        while waiting and len(live) < 2:
            k = waiting.pop(0)
            runner.admit(k)
            live.append(k)
        entries = []
        for j, k in enumerate(live):
            n = min(sizes[(i + 3 * j) % len(sizes)], lens[k] - at[k])
            entries.append(entry(k, toks[k][at[k]:at[k] + n]))
        out = runner.step(entries)
        r = 0
        for e in entries:
            got[e.rid].append(out[r:r + len(e.tokens)])
            r += len(e.tokens)
            at[e.rid] += len(e.tokens)
            if at[e.rid] == lens[e.rid]:
                runner.release(e.rid)
                live.remove(e.rid)
        i += 1
    for k in lens:
        assert_close(torch.cat(got[k]), want[k], dtype)
    runner.manager.check_invariants()


@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_replayed_steps_give_what_plain_launches_give(name):
    """The same requests through steps captured as CUDA graphs (padding requests, the spare state slot) and through
    steps launched kernel by kernel."""
    case, w = for_dtype(CASES[name], torch.bfloat16), make_weights(CASES[name], SEEDS[name])
    toks = {k: random_tokens(n, case["vocab"], seed=n) for k, n in (("a", 70), ("b", 45))}
    outs = []
    for graphs in (False, True):
        runner = make_runner(case, w, torch.bfloat16, use_graphs=graphs)
        assert (runner.graphs is not None) == graphs
        runner.admit("a")
        runner.admit("b")
        rows = [runner.step([entry("a", toks["a"][:40]), entry("b", toks["b"][:33])])]
        for i in range(12):
            rows.append(runner.step([entry("a", [toks["a"][40 + i]]), entry("b", [toks["b"][33 + i]])]))
        rows.append(runner.step([entry("a", toks["a"][52:])]))
        outs.append(torch.cat(rows))
    assert_close(outs[1], outs[0], torch.bfloat16)
    want = torch.cat([pt.forward(case, w, toks["a"])[:40], pt.forward(case, w, toks["b"])[:33]])
    assert_close(outs[1][:73], want, torch.bfloat16)


def test_long_decoding_keeps_state_and_keys():
    case, w = CASE_P, make_weights(CASE_P, 21)
    toks = random_tokens(260, case["vocab"], seed=8)
    want = pt.forward(case, w, toks)
    runner = make_runner(case, w, torch.float32, n_pages=20, max_requests=1, use_graphs=True)
    runner.admit(0)
    rows = [runner.step([entry(0, toks[:5])])]
    for t in toks[5:]:
        rows.append(runner.step([entry(0, [t])]))
    assert rel_err(torch.cat(rows), want) < TOL[torch.float32]
    # the early tokens matter to the last logits: without them the states are other ones
    late = pt.forward(case, w, toks[120:])
    assert rel_err(late[-1], want[-1]) > 1e-3


def write_folder(path, case, w):
    from inferrs_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(case, f)
    write_safetensors(os.path.join(path, "model.safetensors"), [(k, v.to(torch.bfloat16)) for k, v in w.items()])
    return path


def test_greedy_generation_through_the_engine(tmp_path):
    """More requests than slots and few pages: the scheduler admits, cuts prompts into portions, preempts and computes
    again; every request gets the tokens that the plain statement picks."""
    from inferrs_b200.engine.engine import Engine
    from inferrs_b200.sampling.params import SamplingParams
    case, w = CASE_P, make_weights(CASE_P, 31)
    folder = write_folder(str(tmp_path / "m"), case, w)
    eng = Engine(model_dir=folder, dtype="f32", block_size=16, num_blocks=8, max_batch_size=2, max_tokens_per_step=24)
    prompts = [random_tokens(n, case["vocab"], seed=60 + n) for n in (33, 5, 40, 18)]
    n_new = 14
    want = [pt.greedy(case, w, p, n_new) for p in prompts]
    got = eng.generate(prompts, SamplingParams.greedy(max_tokens=n_new))
    eng.runner.manager.check_invariants()
    assert got == want
    assert eng.generate(prompts[:2], SamplingParams.greedy(max_tokens=n_new)) == want[:2]    # slots used before


def test_command_line_with_random_weights_and_with_a_folder(tmp_path, capsys):
    from inferrs_b200 import cli
    path = str(tmp_path / "config.json")
    with open(path, "w") as f:
        json.dump(dict(CASE_P, eos_token_id=5), f)
    common = [path, "--random-weights", "4", "--max-blocks", "32", "--max-batch-size", "2", "--max-tokens", "7",
              "--ignore-eos", "--seed", "3", "--prefill-chunk", "16", "--random-prompt", "45"]
    outs = []
    for _ in range(2):
        assert cli.main(["run"] + common + ["--temperature", "0.8", "--top-k", "20", "--dtype", "bf16"]) == 0
        cap = capsys.readouterr()
        outs.append([int(t) for t in cap.out.split()])
        assert "45 prompt tokens, 7 generated" in cap.err
    assert outs[0] == outs[1] and len(outs[0]) == 7 and all(0 <= t < CASE_P["vocab"] for t in outs[0])
    folder = write_folder(str(tmp_path / "m"), CASE_Q, make_weights(CASE_Q, 5))
    assert cli.main(["bench", folder, "--prompt-len", "30", "--max-tokens", "6", "--runs", "2", "--warmup", "1",
                     "--max-blocks", "32", "--max-batch-size", "2", "--temperature", "0"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["prompt_len"] == 30 and out["prefill_tok_s"] > 0 and out["decode_tok_s"] > 0


def test_trace_replay_of_a_folder(tmp_path):
    case, w = CASE_R, make_weights(CASE_R, 41)
    folder = write_folder(str(tmp_path / "m"), case, w)
    toks = {k: random_tokens(n, case["vocab"], seed=n) for k, n in (("a", 70), ("b", 21))}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks["a"][:50], "want": [0, 49]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks["a"][50:51], "want": [0]},
                                     {"id": "b", "tokens": toks["b"][:19], "want": [18]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": toks["b"][19:], "want": [0, 1]},
                                     {"id": "a", "tokens": toks["a"][51:], "want": [18]}], "end": ["a", "b"]}]
    out_dir = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", out_dir, "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-800:]
    assert p.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    wa, wb = pt.forward(case, w, toks["a"]), pt.forward(case, w, toks["b"])
    read = lambda s: torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{s}.f32"), dtype="<f4").reshape(-1, case["vocab"]).copy())
    assert rel_err(read(0), wa[[0, 49]]) < 2e-4
    assert rel_err(read(1), torch.stack([wa[50], wb[18]])) < 2e-4
    assert rel_err(read(2), torch.stack([wb[19], wb[20], wa[69]])) < 2e-4


# ---------------------------------------------------------------------------------------------------
# keys at the edges of chunks, in the model
# ---------------------------------------------------------------------------------------------------
ONE_ATTENTION = {
    "architecture": "Tikizen", "vocab": 64, "width": 64, "norm": {"eps": 1e-5}, "postln_alpha": 1.0,
    "layers": [{"type": "attention", "mlp": None,
                "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 6.0, "mask": {"size": 48},
                          "rot": None}}],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim", [32, 64, 128])
def test_a_marked_token_is_seen_inside_its_chunk_and_nowhere_else(dim, dtype):
    """One layer of attention without rotation whose keys are the tokens' ids; the query of token 7 asks for token 9,
    and only token 9 has a value: the mark.  Token 9 stands once, at position 200 of a long prompt (chunk 192..239
    of 48).  A token 7 returns the mark if and only if it stands later in the same chunk: at the chunk's last
    position, not at the next chunk's first, not before the mark, not far away.  Whole, cut into portions at odd
    places, and decoded one by one across the chunk's edge."""
    case = json.loads(json.dumps(ONE_ATTENTION))
    case["layers"][0]["mixer"].update(dim=dim, vdim=dim)
    w = make_weights(case, 2)
    width, vocab = 64, 64
    w["embed"], w["embed.norm"] = torch.eye(vocab, width) * 8.0, torch.ones(width)
    pick = torch.zeros(dim, width)
    pick[:min(dim, width)] = torch.eye(width)[:min(dim, width)]
    ask = pick.clone()
    ask[7, 7], ask[9, 7] = 0.0, 1.0                               # token 7 asks for token 9
    w["l0.mix.q"] = torch.cat([ask, ask])
    w["l0.mix.k"] = pick.clone()
    v = torch.zeros(dim, width)
    v[0, 9] = 4.0                                                 # only token 9 has a value
    w["l0.mix.v"] = v
    o = torch.zeros(width, 2 * dim)
    o[63, 0] = 50.0                                               # which goes to channel 63 of the stream
    w["l0.mix.o"] = o
    w["l0.norm1"], w["final.norm"] = torch.ones(width), torch.ones(width)
    w["head"] = torch.eye(vocab, width)
    n, marked_at = 400, 200
    toks = [(11 + i % 20) for i in range(n)]
    toks[marked_at] = 9
    probes = {201: True, 210: True, 239: True, 240: False, 390: False, 191: False, 199: False, 10: False}
    for p in probes:
        toks[p] = 7
    want = pt.forward(case, w, toks)
    assert {p: bool(want[p, 63] > 4.0) for p in probes} == probes       # the plain statement agrees with the story
    runner = make_runner(case, w, dtype, n_pages=60, max_requests=2)
    runner.admit("w")
    got = runner.step([entry("w", toks)])
    runner.admit("c")
    rows, at = [], 0
    for k in cut(235, [64, 2, 48, 31, 90]):                       # portions that end inside and at the edges of chunks
        rows.append(runner.step([entry("c", toks[at:at + k])]))
        at += k
    for t in toks[235:260]:                                       # decoding across the edge 239 | 240
        rows.append(runner.step([entry("c", [t])]))
    rows.append(runner.step([entry("c", toks[260:])]))
    for g in (got, torch.cat(rows)):
        assert_close(g, want, dtype)
        assert {p: bool(g[p, 63] > 4.0) for p in probes} == probes
        assert all(abs(float(g[p, 63])) < 0.5 for p, seen in probes.items() if not seen)


ONE_RETENTION = {
    "architecture": "Tikizen", "vocab": 64, "width": 64, "norm": {"eps": 1e-5}, "postln_alpha": 1.0,
    "layers": [{"type": "retention", "mlp": None,
                "mixer": {"heads": 1, "dim": 32, "vdim": 32, "decay": [1.0]}}],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decay", [1.0, 0.99])
def test_a_marked_token_far_back_is_kept_by_the_state(decay, dtype):
    """One layer of retention without rotation whose keys are the tokens' ids; the query of token 7 asks for token 9,
    and only token 9 has a value: the mark.  Token 9 stands once, at position 5 of a prompt of 400 tokens.  Every
    token 7 after it returns the mark, hundreds of tokens later too (the head is brought to unit size, so a decay
    only weakens what the norm then restores); a token 7 before it does not, and neither does a token 7 early in the
    next request that takes the same state slot."""
    case = json.loads(json.dumps(ONE_RETENTION))
    case["layers"][0]["mixer"]["decay"] = [decay]
    w = make_weights(case, 2)
    width, vocab, dim = 64, 64, 32
    w["embed"], w["embed.norm"] = torch.eye(vocab, width) * 8.0, torch.ones(width)
    pick = torch.eye(width)[:dim].clone()
    ask = pick.clone()
    ask[7, 7], ask[9, 7] = 0.0, 1.0                               # token 7 asks for token 9
    w["l0.mix.q"], w["l0.mix.k"] = ask, pick
    v = torch.zeros(dim, width)
    v[0, 9] = 4.0                                                 # only token 9 has a value
    w["l0.mix.v"] = v
    w["l0.mix.g"] = torch.full((dim, width), 0.25)                # the same gate for every token
    o = torch.zeros(width, dim)
    o[63, 0] = 50.0                                               # the mark goes to channel 63 of the stream
    w["l0.mix.o"] = o
    w["l0.norm1"], w["final.norm"] = torch.ones(width), torch.ones(width)
    w["head"] = torch.eye(vocab, width)
    n, marked_at = 400, 5
    toks = [(11 + i % 20) for i in range(n)]
    toks[marked_at] = 9
    probes = {2: False, 6: True, 17: True, 64: True, 250: True, 399: True}
    for p in probes:
        toks[p] = 7
    want = pt.forward(case, w, toks)
    assert {p: bool(want[p, 63] > 4.0) for p in probes} == probes
    runner = make_runner(case, w, dtype, n_pages=60, max_requests=1)      # one slot: the next request takes it again
    runner.admit("w")
    got = runner.step([entry("w", toks)])
    runner.release("w")
    runner.admit("c")
    rows, at = [], 0
    for k in cut(300, [3, 2, 1, 64, 30, 2, 90]):                  # the mark and the first probes in portions of their own
        rows.append(runner.step([entry("c", toks[at:at + k])]))
        at += k
    for t in toks[300:]:
        rows.append(runner.step([entry("c", [t])]))
    for g in (got, torch.cat(rows)):
        assert_close(g, want, dtype)
        assert {p: bool(g[p, 63] > 4.0) for p in probes} == probes
        assert abs(float(g[2, 63])) < 0.5


# ---------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 90, 1024])
def test_norm_after_the_sum(width, dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(width)
    n, alpha = 7, 2.5
    x = torch.randn(n, width, generator=g) * 3
    delta = torch.randn(n, width, generator=g).to(dtype).float()
    wgt = 1 + 0.2 * torch.randn(width, generator=g)
    want = pt.rms_norm(alpha * x + delta, wgt, 1e-5)
    res, copy = x.cuda().contiguous(), torch.empty((n, width), dtype=dtype, device="cuda")
    kernels.scaled_add_norm(res, act(delta, dtype), alpha, wgt.cuda(), 1e-5, copy, dtype)
    assert rel_err(res, want) < 1e-5
    assert rel_err(copy, want) < (1e-5 if dtype == torch.float32 else 1e-2)
    # nothing to add and no copy: the norm of the embedding
    res = x.cuda().contiguous()
    kernels.scaled_add_norm(res, None, 1.0, wgt.cuda(), 1e-5, None, dtype)
    assert rel_err(res, pt.rms_norm(x, wgt, 1e-5)) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("scaling", [None, (4.0, 64, 16.0, 1.0), (32.0, 8192, 32.0, 1.0)])
def test_rotation_tables_and_heads_as_float(scaling, dtype):
    from inferrs_b200 import kernels
    from inferrs_b200.parts.basic import build_position
    from inferrs_b200.parts.spec import PositionSpec
    from inferrs_b200.runtime import Runtime
    H, D, E, dims, base = 3, 24, 10, 16, 10000.0
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    pos_part = build_position(PositionSpec(kind="rotary_scaled", rot_dim=dims, theta=base, max_positions=3000,
                                           scaling=None if not scaling else tuple(float(v) for v in scaling)),
                              Runtime.cuda(dtype))
    cos, sin, rot_dim = pos_part.tables()
    g = torch.Generator().manual_seed(3)
    positions = [0, 1, 2, 63, 64, 999, 2999]
    n = len(positions)
    src = torch.randn(n, 5 + 2 * H * D + H * E, generator=g).to(dtype)
    dst = torch.full((n, 2 * H * D + H * E + 3), 7.0, dtype=torch.float32, device="cuda")
    slices = ((5, 0, H, D, 1, 1.0), (5 + H * D, H * D, H, D, 1, D ** -0.5), (5 + 2 * H * D, 2 * H * D, H, E, 0, 1.0))
    kernels.heads_to_float(src.cuda(), slices, dst, cos, sin, rot_dim, dev(positions))
    s64 = src.double()
    q = pt.rotate(s64[:, 5:5 + H * D].reshape(n, H, D), torch.tensor(positions), rot)
    k = pt.rotate(s64[:, 5 + H * D:5 + 2 * H * D].reshape(n, H, D), torch.tensor(positions), rot) * D ** -0.5
    assert rel_err(dst[:, :H * D], q.reshape(n, -1)) < 2e-6
    assert rel_err(dst[:, H * D:2 * H * D], k.reshape(n, -1)) < 2e-6
    assert torch.equal(dst[:, 2 * H * D:2 * H * D + H * E].cpu(), src.float()[:, 5 + 2 * H * D:])
    assert bool((dst[:, -3:] == 7.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,dv,rot,ps", [(6, 3, 48, 20, 32, 8), (4, 4, 16, 40, 16, 4), (2, 1, 128, 128, 128, 16),
                                                 (3, 1, 10, 7, 0, 16)])
def test_rotation_then_unit_norm_and_store_with_values_of_their_own_size(nh, nkv, d, dv, rot, ps, dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(d)
    lens, new = [21, 40], [21, 3]
    n = sum(new)
    positions = [p for l, t in zip(lens, new) for p in range(l - t, l)]
    row_request = [r for r, t in enumerate(new) for _ in range(t)]
    n_pages = 8
    table = torch.tensor([[5, 2, -1], [7, 0, 3]], dtype=torch.int32)
    if ps < 16:
        table = torch.arange(2 * 12, dtype=torch.int32).reshape(2, 12)
        n_pages = 24
    qkv = (torch.randn(n, nh * d + nkv * (d + dv), generator=g) * 2).to(dtype)
    half = rot // 2
    cos = sin = None
    if rot:
        ang = torch.arange(64, dtype=torch.float64)[:, None] * (100.0 ** (-torch.arange(half, dtype=torch.float64) / half))
        cos, sin = (torch.cos(ang) * 1.1).float().cuda(), (torch.sin(ang) * 1.1).float().cuda()
    k_pages = torch.zeros((n_pages, nkv, ps, d), dtype=dtype, device="cuda")
    v_pages = torch.zeros((n_pages, nkv, ps, dv), dtype=dtype, device="cuda")
    q_out = torch.empty((n, nh, d), dtype=dtype, device="cuda")
    kernels.qk_norm_rope_store(qkv.cuda(), nh, nkv, d, True, None, None, 1e-5, cos, sin, rot, dev(positions),
                               dev(row_request), table.cuda(), k_pages, v_pages, q_out, norm_q=True, norm_k=True,
                               norm_after_rotation=True)

    def turned(x):                 # [n, heads, d] in float64
        if not rot:
            return x
        c, s = cos.cpu().double()[positions][:, None, :], sin.cpu().double()[positions][:, None, :]
        u, v = x[..., :half], x[..., half:rot]
        return torch.cat([u * c - v * s, v * c + u * s, x[..., rot:]], dim=-1)

    x = qkv.double()
    want_q = pt.rms_unit(turned(x[:, :nh * d].reshape(n, nh, d)), 1e-5)
    want_k = pt.rms_unit(turned(x[:, nh * d:(nh + nkv) * d].reshape(n, nkv, d)), 1e-5)
    want_v = x[:, (nh + nkv) * d:].reshape(n, nkv, dv)
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    assert rel_err(q_out, want_q) < tol
    for row, (p, r) in enumerate(zip(positions, row_request)):
        page = int(table[r, p // ps])
        assert rel_err(k_pages[page, :, p % ps], want_k[row]) < tol
        assert rel_err(v_pages[page, :, p % ps], want_v[row]) < tol


def chunked_attention(q, k, v, positions, scale, chunk):
    """q [n, H, D] at ``positions`` over one request's keys k [T, G, D] and values v [T, G, E], float64."""
    n, H, _ = q.shape
    G = k.shape[1]
    j = torch.arange(k.shape[0])[None, :]
    i = torch.as_tensor(positions)[:, None]
    see = j <= i
    if chunk:
        see = see & ((j // chunk) == (i // chunk))
    out = torch.zeros(n, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        s = (q[:, h].double() @ k[:, h // (H // G)].double().T) * scale
        out[:, h] = torch.softmax(s.masked_fill(~see, float("-inf")), -1) @ v[:, h // (H // G)].double()
    return out.reshape(n, -1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,dv,chunk", [(4, 2, 24, 20, 40), (3, 3, 10, 7, 7), (2, 1, 32, 48, None),
                                                (6, 1, 64, 64, 120), (1, 1, 200, 130, 33)])
def test_generic_attention_with_chunks_and_values_of_their_own_size(nh, nkv, d, dv, chunk, dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(d + dv)
    ps, lens, new = 16, [150, 41, 1], [60, 1, 1]
    pages_per = [(l + ps - 1) // ps for l in lens]
    perm = torch.randperm(sum(pages_per) + 2, generator=g).tolist()
    table = torch.full((3, max(pages_per)), -1, dtype=torch.int32)
    k_pages = torch.full((len(perm), nkv, ps, d), float("nan"))
    v_pages = torch.zeros((len(perm), nkv, ps, dv))
    ks, vs = [], []
    for r, l in enumerate(lens):
        k, v = torch.randn(l, nkv, d, generator=g).to(dtype).float(), torch.randn(l, nkv, dv, generator=g).to(dtype).float()
        ks.append(k)
        vs.append(v)
        for p in range(pages_per[r]):
            page = perm.pop()
            table[r, p] = page
            part = slice(p * ps, min((p + 1) * ps, l))
            k_pages[page, :, :part.stop - part.start] = k[part].transpose(0, 1)
            v_pages[page, :, :part.stop - part.start] = v[part].transpose(0, 1)
    positions = [p for l, t in zip(lens, new) for p in range(l - t, l)]
    row_request = [r for r, t in enumerate(new) for _ in range(t)]
    n = len(positions)
    q = torch.randn(n, nh, d, generator=g).to(dtype).float()
    out = torch.empty((n, nh * dv), dtype=dtype, device="cuda")
    kernels.paged_attention_generic(act(q, dtype), act(k_pages, dtype), act(v_pages, dtype), table.cuda(),
                                    dev(row_request), dev(positions), 0.3, kernels.span_argument(None, chunk), out)
    at = 0
    for r, t in enumerate(new):
        want = chunked_attention(q[at:at + t], ks[r], vs[r], positions[at:at + t], 0.3, chunk)
        assert rel_err(out[at:at + t], want) < (1e-5 if dtype == torch.float32 else 1.5e-2), r
        at += t


@pytest.mark.parametrize("name", ["tcgen05", "pair", "mma", "decode", "generic"])
@pytest.mark.parametrize("chunk", [48, 120, 333])
def test_the_key_just_before_a_chunk_is_not_seen_and_its_first_key_is(name, chunk):
    """Head size 128 in bfloat16: every attention kernel that the engine may pick.  The key just before the row's
    chunk is made to stand out so much that it alone would decide the row if it were admitted; then the chunk's
    first key, which does decide it."""
    import kernel_refs as R
    from test_kernels_gpu import _attention_kernels, _no_error, _paged_setup, rand
    nh, nkv, d, ps, dtype = 8, 2, 128, 16, torch.bfloat16
    lens = [500, 330, 700]
    new = [1, 1, 1] if name == "decode" else [40, 1, 333]
    for inside in (False, True):
        table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 40)
        n = sum(new)
        q = rand((n, nh, d), dtype, 41)
        scale = d ** -0.5 * 4
        rows_last = [sum(new[:r + 1]) - 1 for r in range(len(new))]        # each request's last row
        for r, row in enumerate(rows_last):
            first = ((lens[r] - 1) // chunk) * chunk
            at = first if inside else first - 1
            if at < 0:
                continue
            page, slot = int(table[r, at // ps]), at % ps
            k_pages[page, :, slot, :] = 0
            k_pages[page, :, slot, 0] = 16.0
            v_pages[page, :, slot, :] = 100.0
            q[row, :, :] = 0
            q[row, :, 0] = 16.0
        out = torch.full((n, nh * d), float("nan"), dtype=dtype, device="cuda")
        _attention_kernels(nh, nkv)[name](q, k_pages, v_pages, table, new, positions, row_request, scale, -chunk, out)
        _no_error()
        at = 0
        for r, t in enumerate(new):
            rows = slice(at, at + t)
            pos = positions[rows].tolist()
            js = torch.arange(lens[r])
            pages = table[r, (js // ps).long()].long()
            k = k_pages[pages, :, (js % ps).long(), :].float().cpu()
            v = v_pages[pages, :, (js % ps).long(), :].float().cpu()
            want = chunked_attention(q[rows].float().cpu(), k, v, pos, scale, chunk)
            assert rel_err(out[rows], want) < 2e-2, (r, inside)
            at += t
        for r, row in enumerate(rows_last):
            if ((lens[r] - 1) // chunk) * chunk - (0 if inside else 1) < 0:
                continue
            if inside:
                assert float((out[row].float() - 100.0).abs().max()) < 2.0, "the chunk's first key was not seen"
            else:
                assert float(out[row].float().abs().max()) < 10.0, "the key just before the chunk was seen"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,E,per_token", [(4, 2, 20, 12, True), (1, 1, 128, 64, False), (3, 3, 36, 8, True),
                                                (6, 2, 48, 32, True), (2, 1, 250, 33, False), (4, 4, 64, 64, False),
                                                (16, 2, 128, 128, True)])
@pytest.mark.parametrize("aligned", [False, True])
def test_decay_scan_against_the_recurrence(H, G, D, E, per_token, aligned, dtype):
    """Three requests of unequal length side by side, in two steps, their state slots out of order; keys shared by
    the heads of a group; a decay per head for all tokens or one per token; key sizes that are no multiple of 16 and
    value sizes that are no multiple of 32."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(H * 100 + D)
    slots = [2, 0, 1]
    c0 = 4 if aligned else 1                                  # where q starts in a row: on a 16-byte boundary or not
    ld = (2 * G * D + H * E + c0 + 6) // 4 * 4 + (0 if aligned else 1)
    n_state = H * D * E + 11                                  # the slot holds more than the matrices
    state = torch.zeros((4, n_state), dtype=torch.float32, device="cuda")
    S = [torch.zeros(H, D, E, dtype=torch.float64) for _ in range(3)]
    skip = torch.randn(H, generator=g) if per_token else None
    fixed = torch.rand(H, generator=g) * 0.1 + 0.9
    for lens in ([5, 1, 19], [3, 30, 1], [1, 1, 1]):
        n = sum(lens)
        x = torch.randn(n, ld, generator=g)
        keep = torch.rand(n, H, generator=g) * 0.3 + 0.7
        take = torch.rand(n, H, generator=g) * 2
        gates = torch.cat([keep, take], dim=1).cuda().contiguous()
        out = torch.empty((n, H, E), dtype=torch.float32, device="cuda")
        q_start = dev([0] + list(np.cumsum(lens)))
        kernels.decay_scan(x.cuda(), c0, c0 + G * D, c0 + 2 * G * D, G, gates[:, :H] if per_token else fixed.cuda(),
                           gates[:, H:] if per_token else None, None if skip is None else skip.cuda(), state, q_start,
                           dev(slots), 3, out, D, dtype, max_rows=max(lens))
        at = 0
        for r, n_r in enumerate(lens):
            for t in range(at, at + n_r):
                q = x[t, c0:c0 + G * D].reshape(G, D).double().repeat_interleave(H // G, dim=0)
                k = x[t, c0 + G * D:c0 + 2 * G * D].reshape(G, D).double().repeat_interleave(H // G, dim=0)
                v = x[t, c0 + 2 * G * D:c0 + 2 * G * D + H * E].reshape(H, E).double()
                a = keep[t].double() if per_token else fixed.double()
                b = take[t].double() if per_token else torch.ones(H, dtype=torch.float64)
                S[r] = a[:, None, None] * S[r] + b[:, None, None] * k[:, :, None] * v[:, None, :]
                want = torch.einsum("hde,hd->he", S[r], q)
                if skip is not None:
                    want = want + skip.double()[:, None] * v
                assert rel_err(out[t], want) < 1e-4, (r, t)
            at += n_r
    for r, slot in enumerate(slots):
        assert rel_err(state[slot, :H * D * E].reshape(H, D, E), S[r]) < 1e-4
        assert float(state[slot, H * D * E:].abs().max()) == 0.0     # what lies behind the matrices is not touched
    assert float(state[3].abs().max()) == 0.0           # a slot that no request of the step names is not touched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,C,H", [(4, 50, 3), (1, 8, 1), (2, 130, 5), (7, 33, 2)])
def test_convolution_with_its_state_and_the_gates(taps, C, H, dtype):
    """Requests cut into steps of unequal sizes, among them steps shorter than the convolution's reach: what the
    state keeps must stand in for the rows of earlier steps exactly."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(taps * 10 + C)
    ld, conv_col, dt_col, off = C + H + 9, 4, 4 + C + 2, 13
    w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    dt_bias, a_log = torch.randn(H, generator=g), torch.randn(H, generator=g) * 0.5
    total = {"a": 40, "b": 17}
    proj = {k: torch.randn(n, ld, generator=g).to(dtype) for k, n in total.items()}
    state = torch.zeros((3, off + max(taps - 1, 0) * C + 2), dtype=torch.float32, device="cuda")
    state[:, :off] = 5.0                                          # the matrices' place: not this kernel's
    slot = {"a": 2, "b": 0}
    want = {}
    for k, p in proj.items():
        x = p.double()[:, conv_col:conv_col + C]
        padded = torch.cat([torch.zeros(taps - 1, C, dtype=torch.float64), x])
        acc = b.double()[None, :].expand(total[k], -1).clone()
        for j in range(taps):
            acc = acc + padded[j:j + total[k]] * w.double()[:, j][None, :]
        dt = torch.nn.functional.softplus(p.double()[:, dt_col:dt_col + H] + dt_bias.double())
        want[k] = (acc * torch.sigmoid(acc), torch.exp(-torch.exp(a_log.double()) * dt), dt)
    at = {"a": 0, "b": 0}
    steps = [{"a": 1, "b": 2}, {"a": 1}, {"b": 1, "a": 2}, {"a": 20, "b": 1}, {"b": 13}, {"a": 16}]
    for step in steps:
        keys = list(step)
        rows = torch.cat([proj[k][at[k]:at[k] + step[k]] for k in keys]).cuda().contiguous()
        n = rows.shape[0]
        q_start = dev([0] + list(np.cumsum([step[k] for k in keys])))
        slots = dev([slot[k] for k in keys])
        row_request = dev([i for i, k in enumerate(keys) for _ in range(step[k])])
        out = torch.empty((n, C), dtype=torch.float32, device="cuda")
        gates = torch.empty((n, 2 * H), dtype=torch.float32, device="cuda")
        kernels.conv_silu_gates(rows, conv_col, w.cuda(), b.cuda(), state, off, q_start, slots, row_request, out,
                                dt_col, dt_bias.cuda(), a_log.cuda(), gates)
        kernels.conv_state_shift(rows, conv_col, C, taps, state, off, q_start, slots, len(keys))
        r0 = 0
        for k in keys:
            sl = slice(at[k], at[k] + step[k])
            assert rel_err(out[r0:r0 + step[k]], want[k][0][sl]) < 1e-5, (k, at[k])
            assert rel_err(gates[r0:r0 + step[k], :H], want[k][1][sl]) < 1e-5
            assert rel_err(gates[r0:r0 + step[k], H:], want[k][2][sl]) < 1e-5
            r0 += step[k]
            at[k] += step[k]
    assert at == total
    assert bool((state[:, :off] == 5.0).all()) and float(state[1, off:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("groups,inner", [(1, 48), (2, 192), (3, 45), (12, 96), (2, 2048), (1, 4096), (16, 1024)])
def test_gate_then_norm_in_parts(groups, inner, dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(inner)
    n = 6
    y = torch.randn(n, inner, generator=g) * 3
    wide = torch.randn(n, inner + 9, generator=g).to(dtype)
    wgt = 1 + 0.2 * torch.randn(inner, generator=g)
    z = wide.double()[:, :inner]
    gated = y.double() * z * torch.sigmoid(z)
    want = pt.rms_unit(gated.reshape(n, groups, inner // groups), 1e-5).reshape(n, inner) * wgt.double()
    out = torch.empty((n, inner), dtype=dtype, device="cuda")
    kernels.gate_group_norm(y.cuda(), wide.cuda()[:, :inner], wgt.cuda(), groups, 1e-5, out)
    assert rel_err(out, want) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inner", [37, 64, 1000])
def test_clamped_gate(inner, dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(8)
    gu = (torch.randn(5, 2 * inner, generator=g) * 3).to(dtype)
    lim = 1.5
    gg = torch.clamp(gu.double()[:, :inner], max=lim)
    uu = torch.clamp(gu.double()[:, inner:], min=-lim, max=lim)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1)
    out = torch.empty((5, inner), dtype=dtype, device="cuda")
    kernels.clamped_gate(gu.cuda(), out, lim, 1.702)
    assert rel_err(out, want) < (1e-5 if dtype == torch.float32 else 1e-2)
    assert float(gu.float().max()) > lim and float(gu.float()[:, inner:].min()) < -lim     # the clamps were at work


@pytest.mark.parametrize("ff,shared_ff", [(6, 10), (8, 24)])
@pytest.mark.parametrize("experts,top,shared", [(8, 4, True), (5, 2, False), (3, 3, True), (70, 6, False), (4, 1, True)])
def test_router_weights_and_the_routed_gate(experts, top, shared, ff, shared_ff):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(experts)
    n = 9
    logits = torch.randn(n, experts + int(shared) + 2, generator=g) * 2
    logits[0, 1] = logits[0, 0]                                   # equal logits: the lower index wins
    bias = torch.randn(experts, generator=g)
    z = logits[:, :experts].double() + bias.double()
    best, chosen = torch.topk(z, top, dim=-1)
    want = torch.zeros(n, experts + int(shared), dtype=torch.float64)
    want.scatter_(1, chosen, torch.softmax(best, dim=-1))
    if shared:
        want[:, experts] = torch.sigmoid(logits[:, experts].double())
    got = torch.empty((n, experts + int(shared)), dtype=torch.float32, device="cuda")
    kernels.router_topk(logits.cuda(), bias.cuda(), experts, top, shared, got, torch.float32)
    assert rel_err(got, want) < 1e-5
    assert int((got[:, :experts] > 0).sum()) == n * top
    for dtype in DTYPES:
        inner = experts * ff + (shared_ff if shared else 0)
        gu = torch.randn(n, 2 * inner, generator=g).to(dtype)
        col_expert = torch.tensor([min(j // ff, experts) for j in range(inner)])
        a, b = gu.double()[:, :inner], gu.double()[:, inner:]
        ref = a * torch.sigmoid(a) * b * want[:, col_expert]
        out = torch.empty((n, inner), dtype=dtype, device="cuda")
        kernels.routed_gate(gu.cuda(), got, experts, ff, out)
        assert rel_err(out, ref) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_each_feed_forward_and_mixer_alone_in_a_model_of_one_layer(dtype):
    """Every part as the only layer of a model, against its own function of the plain statement."""
    layers = [CASE_P["layers"][0], CASE_P["layers"][1], CASE_P["layers"][3], CASE_R["layers"][0]]
    for i, layer in enumerate(layers):
        case = {k: v for k, v in (CASE_R if i == 3 else CASE_P).items() if k != "layers"}
        case["layers"] = [layer]
        w = make_weights(case, 50 + i)
        toks = random_tokens(70, case["vocab"], seed=i)
        runner = make_runner(case, w, dtype)
        runner.admit(0)
        got = runner.step([entry(0, toks[:37])])
        got = torch.cat([got, runner.step([entry(0, toks[37:])])])
        assert_close(got, pt.forward(case, w, toks), dtype)
