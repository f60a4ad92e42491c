"""The engine around the kernels: long decoding, the first tokens of a sequence, sharp
attention that shows a missing key, pages of other sizes, sharing and copy-on-write,
a failing step, and the bin/trace_run program itself."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_gpt2
from helpers import ATOL, TINY, Replayer, compare, make_folder, oracle_logits, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {(name, dtype): make_folder(str(tmp_path_factory.mktemp(f"e{name}{dtype}")), raw, seed,
                                       dtype)
            for name, (raw, seed) in TINY.items() for dtype in DTYPES}


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(folders, dtype):
    """A short prompt, then every position up to the model's last one token by token."""
    raw, seed = TINY["B"]
    folder = folders[("B", dtype)]
    ids = random_tokens(raw["n_positions"], raw["vocab_size"], 41)
    oracle = oracle_logits(folder, {"long": ids})
    rp = Replayer(folder, dtype, max_tokens=256)
    rp.step([("long", ids[:3], [0, 1, 2])])
    for i in range(3, len(ids)):
        rp.step([("long", ids[i:i + 1], [0])])
    assert len(rp.rows) == raw["n_positions"]
    compare(rp.rows, oracle, ATOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens(folders, name, dtype):
    """Positions 0, 1, 2: alone, together, and beside another request."""
    raw, seed = TINY[name]
    folder = folders[(name, dtype)]
    prompts = {"x": random_tokens(3, raw["vocab_size"], 1), "y": random_tokens(3, raw["vocab_size"], 2),
               "z": random_tokens(1, raw["vocab_size"], 3)}
    oracle = oracle_logits(folder, prompts)
    rp = Replayer(folder, dtype, max_tokens=256)
    rp.step([("x", prompts["x"][:1], [0])])
    rp.step([("x", prompts["x"][1:2], [0]), ("y", prompts["y"], [0, 1, 2])], end=["y"])
    rp.step([("z", prompts["z"], [0]), ("x", prompts["x"][2:], [0])], end=["x", "z"])
    compare(rp.rows, oracle, ATOL[dtype])


def _sharpen(folder, factor):
    """Scale the query and key parts of every fused QKV matrix so that the softmax is
    peaked: a key that is missed, doubled or taken from a wrong page then changes the
    logits by far more than the tolerance."""
    from safetensors.torch import load_file, save_file
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    d = t["wte.weight"].shape[1]
    for name in list(t):
        if name.endswith("attn.c_attn.weight"):
            w = t[name].float()
            w[:, :2 * d] *= factor
            t[name] = w.to(t[name].dtype)
    save_file(t, path)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page_size", [16, 64, 128])
def test_sharp_attention_across_page_edges(tmp_path, dtype, page_size):
    raw, seed = TINY["B"]
    folder = make_folder(str(tmp_path / "sharp"), raw, seed, dtype)
    _sharpen(folder, 12.0)
    prompts = {"p": random_tokens(200, raw["vocab_size"], 5), "q": random_tokens(131, raw["vocab_size"], 6)}
    oracle = oracle_logits(folder, prompts)
    # the oracle's attention is peaked: the largest weight of late rows is far from uniform
    rp = Replayer(folder, dtype, max_tokens=512, page_size=page_size)
    cuts = {"p": [page_size - 1, 2, page_size, 1, 1, 37], "q": [page_size + 1, 63, 2]}
    at = {"p": 0, "q": 0}
    k = 0
    while any(at[r] < len(prompts[r]) for r in prompts):
        entries = []
        for r in prompts:
            if at[r] >= len(prompts[r]):
                continue
            n = min(cuts[r][k % len(cuts[r])], len(prompts[r]) - at[r])
            entries.append((r, prompts[r][at[r]:at[r] + n], list(range(n))))
            at[r] += n
        k += 1
        rp.step(entries)
    # sharper softmax amplifies rounding of the scores in bfloat16
    compare(rp.rows, oracle, ATOL[dtype] * (3.0 if dtype == "bfloat16" else 1.0))


@pytest.mark.parametrize("dtype", DTYPES)
def test_fork_shares_pages_and_copies_on_write(folders, dtype):
    raw, seed = TINY["A"]
    folder = folders[("A", dtype)]
    base = random_tokens(70, raw["vocab_size"], 8)
    tails = {"root": random_tokens(20, raw["vocab_size"], 9), "kid": random_tokens(25, raw["vocab_size"], 10)}
    prompts = {"root": base + tails["root"], "kid": base + tails["kid"]}
    oracle = oracle_logits(folder, prompts)
    rp = Replayer(folder, dtype, max_tokens=512)
    rp.step([("root", base, list(range(70)))])
    rp.lm.cache.fork("root", "kid", 70)               # 64 + 6 tokens: the tail page is shared
    rp.pos["kid"] = 70
    shared = rp.lm.cache.block_table("kid", 0)
    assert shared == rp.lm.cache.block_table("root", 0)
    rp.step([("kid", tails["kid"][:5], list(range(5))), ("root", tails["root"][:1], [0])])
    # the child copies the shared tail page; the root, appending in the same step while the
    # child's release is still pending, copies too (the original is freed at commit)
    assert 1 <= rp.lm.runner.counters["cow_copies"] <= 2
    assert rp.lm.cache.block_table("kid", 0)[0] == shared[0]          # full page still shared
    assert rp.lm.cache.block_table("kid", 0)[1] != rp.lm.cache.block_table("root", 0)[1]
    rp.step([("kid", tails["kid"][5:], list(range(20))), ("root", tails["root"][1:], list(range(19)))],
            end=["kid", "root"])
    compare(rp.rows, oracle, ATOL[dtype])
    assert rp.lm.cache.free_pages(0) == rp.lm.cache.allocators[0].num_pages


@pytest.mark.parametrize("dtype", DTYPES)
def test_shared_prefix_through_the_entry_point(folders, dtype):
    from pretrained_rstr_b200 import generate_batch, generate_ids, load_lm
    raw, seed = TINY["B"]
    folder = folders[("B", dtype)]
    plain = plain_gpt2.PlainGPT2(folder)
    m = load_lm(folder, gpu=True, dtype=dtype, max_lanes=4, max_batched_tokens=256,
                prefill_chunk=48, share_prefixes=True)
    prefix = random_tokens(150, raw["vocab_size"], 12)
    prompts = [prefix + random_tokens(n, raw["vocab_size"], 13 + n) for n in (5, 17, 1)]
    first = generate_ids(m, prompts[0], 6)
    hits0 = m.stats()["cache"]["prefix_hits"]
    outs = generate_batch(m, prompts, 6)
    assert m.stats()["cache"]["prefix_hits"] >= hits0 + 3 * 2      # two full pages each
    for p, got in zip(prompts, outs):
        want = plain_gpt2.greedy_generate(plain, p, 6)
        if dtype == "float32":
            assert got == want
        else:
            for i, (a, b) in enumerate(zip(got, want)):
                if a != b:
                    row = plain_gpt2.all_logits(plain, p + want[:i])[-1]
                    assert abs(float(row[a] - row[b])) < 3e-2
                    break
    assert outs[0] == first
    m.loaded.cache.check()


def test_failing_step_leaves_the_cache_unchanged(folders):
    """A fault injected on the host after the reservation: the append is aborted, lengths
    and pages are as before, and the same step then succeeds."""
    raw, seed = TINY["A"]
    folder = folders[("A", "float32")]
    ids = random_tokens(80, raw["vocab_size"], 3)
    oracle = oracle_logits(folder, {"f": ids})
    rp = Replayer(folder, "float32", max_tokens=256)
    rp.step([("f", ids[:60], [59])])
    free = rp.lm.cache.free_pages(0)
    rp.lm.runner.fail_next_step = RuntimeError("injected")
    with pytest.raises(RuntimeError, match="injected"):
        rp.lm.runner.step([__import__("pretrained_rstr_b200.engine.batch", fromlist=["Entry"])
                          .Entry("f", ids[60:], [0])])
    assert rp.lm.cache.length("f") == 60 and rp.lm.cache.free_pages(0) == free
    rp.lm.cache.check()
    rp.step([("f", ids[60:], list(range(20)))], end=["f"])
    compare(rp.rows, oracle, ATOL["float32"])


def test_step_refuses_bad_batches(folders):
    from pretrained_rstr_b200.engine.batch import Entry
    from pretrained_rstr_b200.engine.runner import StepError
    raw, seed = TINY["A"]
    rp = Replayer(folders[("A", "float32")], "float32", max_tokens=256)
    rp.lm.cache.open("a")
    run = rp.lm.runner.step
    with pytest.raises(StepError, match="twice"):
        run([Entry("a", [1], []), Entry("a", [2], [])])
    with pytest.raises(StepError, match="vocabulary"):
        run([Entry("a", [raw["vocab_size"]], [])])
    with pytest.raises(StepError, match="wanted place"):
        run([Entry("a", [1, 2], [2])])
    with pytest.raises(StepError, match="positions"):
        run([Entry("a", [1] * (raw["n_positions"] + 1), [])])
    with pytest.raises(StepError, match="the runtime takes"):
        run([Entry("a", [1] * 100, []), Entry("b", [1] * 100, []), Entry("c", [1] * 100, [])])
    with pytest.raises(StepError, match="no tokens"):
        run([Entry("a", [], [])])
    assert rp.lm.cache.length("a") == 0
    rp.lm.cache.check()


def test_inner_width_that_is_no_multiple_of_8(tmp_path):
    """float32 takes any width; the bfloat16 kernels read rows in 16-byte pieces and say so
    when the model is built, not by a wrong result."""
    raw = dict(TINY["A"][0], n_inner=100)
    ids = random_tokens(70, raw["vocab_size"], 3)
    folder = make_folder(str(tmp_path / "f32"), raw, 5, "float32")
    oracle = oracle_logits(folder, {"a": ids})
    rp = Replayer(folder, "float32", max_tokens=128)
    rp.step([("a", ids[:40], list(range(40)))])
    for i in range(40, len(ids)):
        rp.step([("a", ids[i:i + 1], [0])])
    compare(rp.rows, oracle, ATOL["float32"])
    folder16 = make_folder(str(tmp_path / "bf16"), raw, 5, "bfloat16")
    with pytest.raises(ValueError, match="multiple of 8"):
        Replayer(folder16, "bfloat16", max_tokens=128)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(tmp_path, dtype):
    """bin/trace_run as a user runs it: JSON lines in, <step>.f32 files and 'done' lines out."""
    raw, seed = TINY["A"]
    folder = make_folder(str(tmp_path / "model"), raw, seed, dtype)
    a, b = random_tokens(70, raw["vocab_size"], 1), random_tokens(9, raw["vocab_size"], 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [0, 39]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[40:66], "want": []},
                                {"id": "b", "tokens": b[:2], "want": [1]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[2:], "want": [6]}], "end": ["b"]},
        {"step": 7, "entries": [{"id": "a", "tokens": a[66:], "want": [0, 1, 2, 3]}], "end": ["a"]},
    ]
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
         "--out", str(out), "--max-tokens", "192"],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
        timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == \
        ["done 0", "done 1", "done 2", "done 7"]
    oracle = oracle_logits(folder, {"a": a, "b": b})
    import numpy as np
    vocab = raw["vocab_size"]
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, vocab))
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, vocab))
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, vocab))
    got7 = torch.from_numpy(np.fromfile(out / "7.f32", dtype="<f4").reshape(-1, vocab))
    assert got0.shape[0] == 2 and got1.shape[0] == 1 and got2.shape[0] == 1 and got7.shape[0] == 4
    # beside every file of logits, an index of its rows by (request, position)
    index = {s: json.loads((out / f"{s}.json").read_text()) for s in (0, 1, 2, 7)}
    assert index[0] == {"step": 0, "vocab": vocab, "rows": [["a", 0], ["a", 39]]}
    assert index[1]["rows"] == [["b", 1]] and index[2]["rows"] == [["b", 8]]
    assert index[7]["rows"] == [["a", 66], ["a", 67], ["a", 68], ["a", 69]]
    tol = ATOL[dtype]
    assert float((got0 - oracle["a"][[0, 39]]).abs().max()) <= tol
    assert float((got1 - oracle["b"][[1]]).abs().max()) <= tol
    assert float((got2 - oracle["b"][[8]]).abs().max()) <= tol
    assert float((got7 - oracle["a"][66:70]).abs().max()) <= tol


def _decode_steps(folder, raw, graphs, n_req):
    """A prompt step of `n_req` requests, then five decode steps of all of them, replayed as CUDA
    graphs from the third on (`graphs`) or launched kernel by kernel."""
    lengths = [raw["n_positions"] - 6, 70, 9, 130, 33, 64, 65, 200][:n_req]
    prompts = {f"d{i}": random_tokens(n, raw["vocab_size"], 50 + i) for i, n in enumerate(lengths)}
    rp = Replayer(folder, "bfloat16", max_tokens=sum(-(-n // 64) * 64 for n in lengths),
                  max_requests=8, max_batched_tokens=2048)
    rp.lm.runner.use_graphs = graphs
    rp.step([(r, ids[:len(ids) - 5], [len(ids) - 6]) for r, ids in prompts.items()])
    for k in range(5, 0, -1):
        rp.step([(r, ids[len(ids) - k:len(ids) - k + 1], [0]) for r, ids in prompts.items()])
    return rp, prompts


@pytest.mark.parametrize("n_req", [1, 3, 8])
def test_decode_graphs_equal_kernel_by_kernel(folders, n_req):
    """Decode steps replayed as CUDA graphs (planned with the capacities of their shape: the
    longest context, padded rows) give the logits of the same steps launched kernel by kernel,
    to rounding, and both match the plain implementation."""
    raw, seed = TINY["C"]
    folder = folders[("C", "bfloat16")]
    results = {}
    for graphs in (True, False):
        rp, prompts = _decode_steps(folder, raw, graphs, n_req)
        assert bool(rp.lm.runner._graphs) == graphs
        compare(rp.rows, oracle_logits(folder, prompts), ATOL["bfloat16"])
        results[graphs] = rp.rows
    for key, row in results[True].items():
        assert float((row - results[False][key]).abs().max()) <= 2e-3


def _run_cli(*args, stdin=None):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run([sys.executable, "-m", "pretrained_rstr_b200", *args], input=stdin,
                          capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    return proc.stdout


@pytest.mark.parametrize("size,seed", [("tiny-a", 0), ("tiny-b", 1)])
def test_command_line_random_then_generate(tmp_path, size, seed):
    """``python -m pretrained_rstr_b200 random`` writes a model folder, ``generate`` prints one
    JSON object with the generated ids: greedy in float32 they are the plain implementation's;
    ``generate --random SIZE`` makes the same weights itself and gives the same ids."""
    folder = str(tmp_path / "model")
    made = json.loads(_run_cli("random", "--out", folder, "--size", size, "--seed", str(seed)))
    assert made["out"] == folder and made["config"]["architectures"] == ["GPT2LMHeadModel"]
    prompt = random_tokens(11, made["config"]["vocab_size"], 21)
    ids = ",".join(str(t) for t in prompt)
    out = json.loads(_run_cli("generate", "--model", folder, "--ids", ids, "--n", "9",
                              "--dtype", "float32").strip().splitlines()[-1])
    want = plain_gpt2.greedy_generate(plain_gpt2.PlainGPT2(folder), prompt, 9)
    assert out["prompt"] == prompt and out["generated"] == want
    again = json.loads(_run_cli("generate", "--random", size, "--weights-seed", str(seed), "--ids", ids,
                                "--n", "9", "--dtype", "float32").strip().splitlines()[-1])
    assert again["generated"] == want
    sampled = json.loads(_run_cli("generate", "--model", folder, "--ids", ids, "--n", "9", "--dtype",
                                  "float32", "--temperature", "0.8", "--seed", "7")
                         .strip().splitlines()[-1])
    assert sampled["generated"] == plain_gpt2.sample_generate(plain_gpt2.PlainGPT2(folder), prompt, 9,
                                                              0.8, None, None, 7)


def test_replay_with_random_weights_and_six_live_requests(tmp_path):
    """``replay --random SIZE --seed S`` makes its own model; ``--max-requests`` lifts the
    default of four live requests."""
    raw, seed = TINY["A"]
    folder = make_folder(str(tmp_path / "same"), raw, seed, "float32")     # what --random tiny-a --seed 0 makes
    prompts = {f"r{i}": random_tokens(7 + 3 * i, raw["vocab_size"], 60 + i) for i in range(6)}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": ids[:-1], "want": []} for r, ids in prompts.items()],
              "end": []},
             {"step": 1, "entries": [{"id": r, "tokens": ids[-1:], "want": [0]} for r, ids in prompts.items()],
              "end": list(prompts)}]
    out = tmp_path / "out"
    text = "".join(json.dumps(s) + "\n" for s in steps)
    done = _run_cli("replay", "--random", "tiny-a", "--seed", "0", "--dtype", "float32", "--out", str(out),
                    "--max-tokens", str(6 * 64), "--max-requests", "6", stdin=text)
    assert [l for l in done.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    import numpy as np
    got = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(6, raw["vocab_size"]))
    index = json.loads((out / "1.json").read_text())
    oracle = oracle_logits(folder, prompts)
    for row, (rid, pos) in zip(got, index["rows"]):
        assert pos == len(prompts[rid]) - 1
        assert float((row - oracle[rid][pos]).abs().max()) <= ATOL["float32"]
    # with the default of four, the fifth live request is refused
    env = dict(os.environ, PYTHONPATH=ROOT)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                           "--dtype", "float32", "--out", str(tmp_path / "o2"), "--max-tokens", "384"],
                          input=text, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode != 0 and "requests" in proc.stderr
