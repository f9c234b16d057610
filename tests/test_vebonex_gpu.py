"""The Vebonex design in the engine against its plain statement: every kernel alone, whole prompts, every way of
cutting a request into steps, batches, slots and pages used again, long decoding, and greedy generation through the
engine's own entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_vebonex as pv
from helpers import cut, random_tokens, rel_err
from vebonex_cases import CASE_P, CASE_Q, CASE_R, CASES, make_weights

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-4, torch.bfloat16: 5e-2}
SEEDS = {"P": 11, "Q": 12, "R": 13, "S": 14}


def assert_close(got, want, dtype):
    """float32: every row within 2e-4 of its largest value.  bfloat16: rounding is amplified without bound where a
    head's output is nearly zero before it is brought to unit size (such rows are a hundred times worse than the
    others in float32 too), so the rows are judged together: their median error and the nineteenth of twenty."""
    if dtype == torch.float32:
        assert rel_err(got, want) < TOL[dtype]
        return
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape and bool(torch.isfinite(got).all())
    err = (got - want).abs().amax(dim=1) / want.abs().amax(dim=1).clamp_min(1e-30)
    assert float(err.median()) < 2e-2, float(err.median())
    assert float(torch.quantile(err, 0.95)) < TOL[dtype], float(torch.quantile(err, 0.95))


def on_device(w, dtype):
    return {k: v.to(dtype).cuda() for k, v in w.items()}


def make_runner(case, w, dtype, n_pages=24, max_requests=3, page_size=16, use_graphs=False):
    from inferrs_b200.engine.loading import spec_from_config
    from inferrs_b200.engine.runner import ModelRunner
    from inferrs_b200.runtime import Runtime
    spec, _ = spec_from_config(case)
    rt = Runtime.cuda(dtype)
    return ModelRunner(spec, on_device(w, dtype), rt, page_size=page_size, n_pages=n_pages, max_requests=max_requests,
                       use_graphs=use_graphs)


def entry(rid, tokens, want=None):
    from inferrs_b200.engine.batch import StepEntry
    return StepEntry(rid, tokens, list(range(len(tokens))) if want is None else want)


# ---------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_whole_prompt_and_every_cutting_match_the_plain_statement(name, dtype):
    case, w = CASES[name], make_weights(CASES[name], SEEDS[name])
    toks = random_tokens(75, case["vocab"], seed=3)
    want = pv.forward(case, w, toks)
    runner = make_runner(case, w, dtype)
    runner.admit("whole")
    got = runner.step([entry("whole", toks)])
    assert_close(got, want, dtype)
    runner.release("whole")
    # one token a step from an empty cache: the first tokens of a sequence, and decoding through cache and state
    runner.admit("single")
    rows = [runner.step([entry("single", [t])]) for t in toks[:40]]
    assert_close(torch.cat(rows), want[:40], dtype)
    runner.release("single")
    # portions of changing size, down to two tokens and one, another request's portions beside them
    other = random_tokens(40, case["vocab"], seed=4)
    want_other = pv.forward(case, w, other)
    runner.admit("cut")
    runner.admit("other")
    at, o_at, rows, o_rows = 0, 0, [], []
    for n in cut(len(toks), [7, 2, 30, 1, 1, 2, 17, 3]):
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


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_unequal_requests_in_one_batch_slots_and_pages_used_again(name, dtype):
    """Two state slots and pages for two requests; five requests of unequal length take turns, decoding side by side
    with portions of the next ones.  Every request must give what it gives alone (the plain statement knows no
    batches, slots or pages)."""
    case, w = CASES[name], make_weights(CASES[name], SEEDS[name])
    lens = {"a": 50, "b": 23, "c": 64, "d": 9, "e": 37}
    toks = {k: random_tokens(n, case["vocab"], seed=ord(k)) for k, n in lens.items()}
    want = {k: pv.forward(case, w, t) for k, t in toks.items()}
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
    case, w = CASES[name], make_weights(CASES[name], SEEDS[name])
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
    want = torch.cat([pv.forward(case, w, toks["a"])[:40], pv.forward(case, w, toks["b"])[:33]])
    assert_close(outs[1][:73], want, torch.bfloat16)


def test_long_decoding_keeps_state_and_latents():
    case, w = CASE_P, make_weights(CASE_P, 21)
    toks = random_tokens(260, case["vocab"], seed=8)
    want = pv.forward(case, w, toks)
    runner = make_runner(case, w, torch.float32, n_pages=20, max_requests=1, use_graphs=True)
    runner.admit(0)
    rows = [runner.step([entry(0, toks[:5])])]
    for t in toks[5:]:
        rows.append(runner.step([entry(0, [t])]))
    assert rel_err(torch.cat(rows), want) < TOL[torch.float32]
    # the early tokens matter to the last logits: without them the state and the latents are other ones
    late = pv.forward(case, w, toks[100:])
    assert rel_err(late[-1], want[-1]) > 1e-2


def write_folder(path, case, w):
    from inferrs_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    config = json.loads(json.dumps(case))
    for layer in config["layers"]:
        layer["mixer"].pop("a_rank", None)       # a folder gives this size by the tensor's shape
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f)
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
    want = [pv.greedy(case, w, p, n_new) for p in prompts]
    got = eng.generate(prompts, SamplingParams.greedy(max_tokens=n_new))
    eng.runner.manager.check_invariants()
    assert got == want
    assert eng.generate(prompts[:2], SamplingParams.greedy(max_tokens=n_new)) == want[:2]    # slots used before


def test_command_line_with_random_weights_and_with_a_folder(tmp_path, capsys):
    """``run --random-weights`` takes the design's config.json (the size that a folder gives by a tensor's shape is a
    key then); sampling with a seed gives the same tokens twice; ``bench`` runs a folder."""
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
    toks = {k: random_tokens(n, case["vocab"], seed=n) for k, n in (("a", 40), ("b", 21))}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks["a"][:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks["a"][30:31], "want": [0]},
                                     {"id": "b", "tokens": toks["b"][:19], "want": [18]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": toks["b"][19:], "want": [0, 1]},
                                     {"id": "a", "tokens": toks["a"][31:], "want": [8]}], "end": ["a", "b"]}]
    out_dir = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", out_dir, "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-800:]
    assert p.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    wa, wb = pv.forward(case, w, toks["a"]), pv.forward(case, w, toks["b"])
    read = lambda s: torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{s}.f32"), dtype="<f4").reshape(-1, case["vocab"]).copy())
    assert rel_err(read(0), wa[[0, 29]]) < 2e-4
    assert rel_err(read(1), torch.stack([wa[30], wb[18]])) < 2e-4
    assert rel_err(read(2), torch.stack([wb[19], wb[20], wa[39]])) < 2e-4


# ---------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------
def act(x, dtype):
    return x.to(dtype).cuda().contiguous()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("streams,groups,width", [(1, 1, 48), (2, 4, 64), (3, 3, 96), (8, 2, 520)])
def test_stream_update_read_and_norm_in_groups(streams, groups, width, dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(streams * 7 + groups)
    n = 9
    x = torch.randn(n, streams, width, generator=g) * 3
    delta = torch.randn(n, width, generator=g).to(dtype).float()
    mix = torch.eye(streams) + 0.3 * torch.randn(streams, streams, generator=g)
    gain, read = torch.randn(streams, generator=g), torch.randn(streams, generator=g)
    wgt = (1 + 0.2 * torch.randn(width, generator=g)).to(dtype).float()
    new = torch.einsum("st,nsw->ntw", mix, x) + gain[None, :, None] * delta[:, None, :]
    want = pv.grouped_norm(torch.einsum("t,ntw->nw", read, new), wgt, groups, 1e-5)
    res = x.cuda().contiguous()
    out = torch.empty((n, width), dtype=dtype, device="cuda")
    kernels.stream_add_norm(res, act(delta, dtype), mix.cuda(), gain.cuda(), read.cuda(), act(wgt, dtype), groups, 1e-5, out)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert rel_err(out, want) < tol
    assert rel_err(res, new) < 1e-6                     # the streams are written back in float32
    # chosen rows, nothing pending, the plain sum: the last norm of a model; nothing is written back
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    before = res.clone()
    out = torch.empty((3, width), dtype=dtype, device="cuda")
    kernels.stream_add_norm(res, None, None, None, None, act(wgt, dtype), groups, 1e-5, out, rows)
    assert rel_err(out, pv.grouped_norm(new.sum(1)[[7, 0, 3]], wgt, groups, 1e-5)) < tol
    assert torch.equal(res, before)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_with_positions_fills_every_stream(dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(1)
    table, pos = torch.randn(50, 40, generator=g).to(dtype), torch.randn(30, 40, generator=g).to(dtype)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device="cuda")
    where = torch.tensor([0, 29, 7, 8], dtype=torch.int32, device="cuda")
    out = torch.empty((4, 3, 40), dtype=torch.float32, device="cuda")
    kernels.embedding_streams(table.cuda(), ids, pos.cuda(), where, out, dtype)
    want = table.float()[ids.cpu().long()] + pos.float()[where.cpu().long()]
    assert all(torch.equal(out[:, s].cpu(), want) for s in range(3))


@pytest.mark.parametrize("dtype", DTYPES)
def test_polynomial_activation_with_unit_rms_terms(dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(2)
    z = (torch.randn(6, 200, generator=g) * 2).to(dtype)
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1])
    out = torch.empty((6, 200), dtype=dtype, device="cuda")
    kernels.poly_norm(z.cuda(), coef.cuda(), 1e-6, out)
    assert rel_err(out, pv.poly_norm_act(z.float(), coef, 1e-6)) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mode,H,D,E", [("decay", 2, 40, 10), ("decay", 1, 128, 64), ("gates", 3, 16, 36),
                                         ("gates", 1, 200, 7)])
def test_scan_kernel_against_the_recurrence(mode, H, D, E, dtype):
    """Three requests of unequal length side by side, in two steps, their state slots out of order; key sizes that
    are no multiple of 32 and value sizes that are no multiple of four."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(H * 100 + D)
    lens1, lens2, slots = [5, 1, 19], [3, 30, 1], [2, 0, 1]
    hd, he = H * D, H * E
    ld = 2 * hd + he + 5                                     # the projection is wider than what the scan reads
    tau, cap = 4.0, 6.0
    n_state = H * E * D + (H * D + H if mode == "gates" else 0)
    state = torch.zeros((4, n_state), dtype=torch.float32, device="cuda")
    ref = [None, None, None]
    for lens in (lens1, lens2):
        n = sum(lens)
        proj = (torch.randn(n, ld, generator=g)).to(dtype).float()
        gw = H * D if mode == "decay" else 2 * H
        gates = torch.randn(n, gw, generator=g) * 2
        bias = torch.randn(gw, generator=g) + 1.0
        out = torch.empty((n, H, E), dtype=torch.float32, device="cuda")
        q_start = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device="cuda")
        kernels.linear_scan(kernels.SCAN_CHANNEL_DECAY if mode == "decay" else kernels.SCAN_SCALAR_GATES,
                            act(proj, dtype), 0, hd, 2 * hd, gates.cuda(), bias.cuda(), tau if mode == "decay" else cap,
                            D ** -0.5, state, q_start, torch.tensor(slots, dtype=torch.int32, device="cuda"), 3, out, D)
        at = 0
        for r, n_r in enumerate(lens):
            rows = slice(at, at + n_r)
            q = proj[rows, :hd].reshape(n_r, H, D).double() * D ** -0.5
            k = proj[rows, hd:2 * hd].reshape(n_r, H, D).double()
            v = proj[rows, 2 * hd:2 * hd + he].reshape(n_r, H, E).double()
            if mode == "decay":
                alpha = torch.sigmoid((gates[rows] + bias).double()).pow(1 / tau).reshape(n_r, H, D)
                want, ref[r] = pv.gla_scan(q, k, v, alpha, ref[r])
            else:
                pre = (gates[rows] + bias).double()
                li = pv.soft_cap(pre[:, :H], cap)
                lf = torch.nn.functional.logsigmoid(pv.soft_cap(pre[:, H:], cap))
                want, ref[r] = pv.mlstm_scan(q, k, v, li, lf, ref[r])
            assert rel_err(out[rows], want) < 1e-4, (r, lens)
            at += n_r
    # the state that the kernel leaves: S as [H, D, E]
    for r, slot in enumerate(slots):
        S = ref[r] if mode == "decay" else ref[r][0]
        assert rel_err(state[slot, :H * E * D].reshape(H, D, E), S) < 1e-4
    assert float(state[3].abs().max()) == 0.0           # a slot that no request of the step names is not touched


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_norm_and_gate(dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(5)
    n, H, E = 7, 3, 20
    o = torch.randn(n, H, E, generator=g) * 4
    wide = torch.randn(n, 11 + H * E, generator=g).to(dtype)
    gate = wide.float()[:, 11:]
    for weight, normed, kind in ((torch.randn(E, generator=g), True, "silu"), (torch.randn(H * E, generator=g), True, "sigmoid"),
                                 (None, False, "sigmoid")):
        w = None if weight is None else weight.to(dtype)
        x = pv.unit_rms(o, 1e-5) if normed else o
        if w is not None:
            x = x * (w.float() if w.numel() == E else w.float().reshape(H, E))
        gg = torch.nn.functional.silu(gate) if kind == "silu" else torch.sigmoid(gate)
        want = x.reshape(n, H * E) * gg
        out = torch.empty((n, H * E), dtype=dtype, device="cuda")
        kernels.head_norm_gate(o.cuda(), wide.cuda()[:, 11:], None if w is None else w.cuda(), normed,
                               kernels.GATE_SILU if kind == "silu" else kernels.GATE_SIGMOID, 1e-5, out)
        assert rel_err(out, want) < (1e-5 if dtype == torch.float32 else 1e-2)
        # a head-major input [H, n, E] read in place
        hm = o.transpose(0, 1).contiguous().cuda()
        kernels.head_norm_gate(hm.transpose(0, 1), wide.cuda()[:, 11:], None if w is None else w.cuda(), normed,
                               kernels.GATE_SILU if kind == "silu" else kernels.GATE_SIGMOID, 1e-5, out)
        assert rel_err(out, want) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_batched_products_per_head(dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(6)
    n, H, K, M = 21, 5, 24, 40
    x = torch.randn(n, H * K, generator=g).to(dtype)
    w = (torch.randn(H, M, K, generator=g) / K ** 0.5).to(dtype)
    out = torch.empty((H, n, M), dtype=dtype, device="cuda")
    kernels.batched_linear(x.cuda().view(n, H, K).transpose(0, 1), w.cuda(), out, dtype)
    want = torch.einsum("nhk,hmk->hnm", x.float().reshape(n, H, K), w.float())
    assert rel_err(out, want) < (1e-5 if dtype == torch.float32 else 1e-2)


def latent_mix(q_lat, c, scale, positions, window=None):
    """out[h, i] = sum_j softmax_j(scale * q_lat[h, i] . c_j) c_j over the j that position positions[i] sees."""
    s = torch.einsum("hir,jr->hij", q_lat, c) * scale
    j = torch.arange(c.shape[0])[None, :]
    i = torch.as_tensor(positions)[:, None]
    hidden = (j > i) if window is None else ((j > i) | (j <= i - window))
    return torch.einsum("hij,jr->hir", torch.softmax(s.masked_fill(hidden, float("-inf")), -1), c)


def paged_latents(c_per_request, page_size, n_pages, dtype, seed):
    """Latents laid into pages in a shuffled order; pages that belong to nobody hold NaN."""
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g).tolist()
    R = c_per_request[0].shape[1]
    plane = torch.full((n_pages, page_size, R), float("nan"))
    width = max((c.shape[0] + page_size - 1) // page_size for c in c_per_request)
    table = torch.full((len(c_per_request), width), -1, dtype=torch.int32)
    for r, c in enumerate(c_per_request):
        for p in range((c.shape[0] + page_size - 1) // page_size):
            page = order.pop()
            table[r, p] = page
            part = c[p * page_size:(p + 1) * page_size]
            plane[page, :part.shape[0]] = part
    return plane.to(dtype).cuda(), table.cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,R,window,slices", [(3, 36, None, 1), (18, 70, None, 1), (2, 130, 40, 1), (5, 300, None, 4),
                                                (1, 512, 100, 3), (17, 24, None, 7),
                                                # ranks that the tensor-core form of the bfloat16 build takes
                                                (6, 96, None, 1), (16, 128, None, 1), (3, 64, 40, 2), (40, 256, None, 3),
                                                (33, 32, 70, 5), (16, 512, None, 2), (5, 64, 33, 1), (16, 512, None, 1)])
def test_latent_attention_kernel(H, R, window, slices, dtype):
    """A portion of one request (its later tokens are in the cache already and must stay unseen), a single token of
    another with many keys, and a first token; shuffled pages."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(H + R)
    page = 16
    held = [200, 333, 1]                                   # tokens in the cache once the step's latents are written
    rows_of = [list(range(150, 200)), [332], [0]]          # the positions of the step's rows
    c = [(torch.randn(n, R, generator=g)).to(dtype).float() for n in held]
    plane, table = paged_latents(c, page, 40, dtype, seed=R)
    positions = [p for rows in rows_of for p in rows]
    row_request = [r for r, rows in enumerate(rows_of) for _ in rows]
    n = len(positions)
    q_lat = (torch.randn(H, n, R, generator=g) * 1.5).to(dtype).float()
    scale = 0.6 / R ** 0.5
    # once row by row, once (one slice) with the rows cut into tiles of two tokens of one request, one place of the
    # list empty: the form that prompt portions take on the tensor cores
    tile_req, tile_row0, starts = [], [], [0]
    for r, rows in enumerate(rows_of):
        tile_req += [r] * ((len(rows) + 1) // 2)
        tile_row0 += list(range(starts[-1], starts[-1] + len(rows), 2))
        starts.append(starts[-1] + len(rows))
    tile_req.insert(3, -1)
    tile_row0.insert(3, 0)
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    tiles = (dev(tile_req), dev(tile_row0), len(tile_req), dev(starts))
    for use_tiles in ([False, True] if slices == 1 else [False]):
        out = torch.full((H, n, R), float("nan"), dtype=dtype, device="cuda")
        kernels.latent_attention(act(q_lat, dtype), plane, table, dev(row_request), dev(positions), scale, window, out,
                                 slices, tiles if use_tiles else None)
        at = 0
        for r, rows in enumerate(rows_of):
            want = latent_mix(q_lat[:, at:at + len(rows)], c[r], scale, rows, window)
            assert rel_err(out[:, at:at + len(rows)], want) < (2e-5 if dtype == torch.float32 else 2e-2), (r, use_tiles)
            at += len(rows)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("R", [48, 64])
@pytest.mark.parametrize("slices", [1, 5])
def test_latent_attention_sees_exactly_its_keys(slices, R, dtype):
    """One latent of the cache is made to stand out (a large multiple of the query's direction), so that whoever
    sees it returns it: a key far back among hundreds, keys at page borders, the row's own key, the key just after
    it (a later token of the same portion), and with a window the keys just inside and just outside it."""
    from inferrs_b200 import kernels
    H, page, n_keys, window = 2, 16, 400, 64
    g = torch.Generator().manual_seed(9)
    direction = torch.nn.functional.normalize(torch.randn(R, generator=g), dim=0)
    base = (0.1 * torch.randn(n_keys, R, generator=g))
    pos = 300
    cases = [(3, None, True), (15, None, True), (16, None, True), (17, None, True), (pos, None, True),
             (pos + 1, None, False), (pos - window + 1, window, True), (pos - window, window, False),
             (pos - window - 1, window, False), (pos - 1, window, True), (288, None, True), (287, window, True)]
    for j, win, seen in cases:
        c = base.clone()
        c[j] = 8.0 * direction
        c = c.to(dtype).float()
        plane, table = paged_latents([c], page, 30, dtype, seed=j)
        q_lat = (direction[None, None, :] * torch.tensor([6.0, 9.0])[:, None, None]).to(dtype).float()       # [H, 1, R]
        out = torch.empty((H, 1, R), dtype=dtype, device="cuda")
        kernels.latent_attention(act(q_lat, dtype), plane, table, torch.zeros(1, dtype=torch.int32, device="cuda"),
                                 torch.tensor([pos], dtype=torch.int32, device="cuda"), 1.0, win, out, slices)
        want = latent_mix(q_lat, c, 1.0, [pos], win)
        assert rel_err(out, want) < (1e-4 if dtype == torch.float32 else 2e-2), (j, win)
        stands_out = float((out.float().cpu()[0, 0] @ direction)) > 4.0
        assert stands_out == seen, (j, win)
