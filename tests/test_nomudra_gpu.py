"""Nomudra through the engine against the plain model (float64): the same requests whole, with their last tokens
decoded one by one, in portions down to two tokens, and mixed with other requests in a pool so small that pages and
state slots are used again; long decoding from a single token; greedy generation through ``LLM.generate`` and the
scheduler, and through the command line.  Small configurations that differ in every size, in the order of their layers
and in every option: chunks smaller and larger than a page and no chunks at all, rotation of a part of the head or of
all of it, one key/value head or as many as query heads, one mLSTM head or several with key and value heads of unequal
size, a small and a large gate cap, routers with and without groups and identity experts, top 1 and top = all, layers
without a feed-forward, sizes that are no multiple of 8."""
import json
import os

import numpy as np
import pytest
import torch

import plain_nomudra as pn
import trace_tools as tt

pytestmark = pytest.mark.gpu


def attn(heads, kv, dim, chunk, rot_dims, base, scale):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale, rot=dict(base=base, dims=rot_dims),
                mask=None if chunk is None else dict(size=chunk))


def mlstm(heads, dim, vdim, cap):
    return dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap)


def moe(experts, identity, top, count, keep, ff, limit, shared_ff, shared_limit):
    return dict(kind="moe", router=dict(experts=experts, identity=identity, top=top, groups=dict(count=count, keep=keep)),
                expert=dict(ff=ff, limit=limit), shared=dict(ff=shared_ff, limit=shared_limit))


NOM_A = dict(architecture="Nomudra", vocab=300, width=128, norm=dict(eps=1e-5), layers=[
    dict(type="attention", mixer=attn(4, 2, 32, 24, 16, 10000.0, 0.2), mlp=moe(6, 2, 2, 4, 2, 48, 1.0, 64, 2.5)),
    dict(type="mlstm", mixer=mlstm(3, 24, 40, 10.0), mlp=None),
    dict(type="attention", mixer=attn(2, 1, 64, 7, 64, 500.0, 0.125), mlp=moe(5, 0, 5, 1, 1, 40, 3.0, 40, 0.5)),
])
NOM_B = dict(architecture="Nomudra", vocab=211, width=96, norm=dict(eps=1e-6), layers=[
    dict(type="mlstm", mixer=mlstm(1, 72, 16, 15.0), mlp=moe(3, 1, 1, 2, 2, 32, 1.5, 16, 2.0)),
    dict(type="mlstm", mixer=mlstm(4, 16, 48, 4.0), mlp=None),
    dict(type="attention", mixer=attn(6, 6, 16, 33, 8, 1000000.0, 0.3), mlp=moe(8, 4, 3, 3, 1, 24, 2.0, 56, 1.0)),
    dict(type="attention", mixer=attn(3, 1, 48, None, 48, 10000.0, 0.15), mlp=None),
])
# sizes that are no multiple of 8 anywhere: every product and the attention take their general paths
NOM_C = dict(architecture="Nomudra", vocab=97, width=100, norm=dict(eps=1e-6), layers=[
    dict(type="attention", mixer=attn(3, 1, 20, 50, 10, 20000.0, 0.25), mlp=moe(4, 1, 2, 5, 3, 36, 1.2, 28, 1.8)),
    dict(type="mlstm", mixer=mlstm(2, 34, 38, 8.0), mlp=moe(2, 0, 1, 2, 1, 20, 2.0, 12, 2.0)),
])
MODELS = {"A": (NOM_A, 21), "B": (NOM_B, 22), "C": (NOM_C, 23)}
LENGTHS = (70, 41, 97, 2, 33, 129, 1, 9, 55)
F32_TOL = 1e-4          # float32 sums in another order than float64
BF16_TOL = 0.05         # activations rounded to 8 bits of mantissa after every op


def write_model(folder, cfg, seed):
    from safetensors.torch import save_file
    w = pn.random_weights(cfg, seed)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(folder, "model.safetensors"))
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return {k: v.to(torch.float64) for k, v in w.items()}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, seed) in MODELS.items():
        d = str(tmp_path_factory.mktemp(f"nomudra_{name}"))
        out[name] = (d, cfg, write_model(d, cfg, seed))
    return out


def requests_for(name):
    cfg, seed = MODELS[name]
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(LENGTHS)}


@pytest.fixture(scope="module")
def references(models):
    return {name: {rid: pn.forward(cfg, w, t).numpy() for rid, t in requests_for(name).items()}
            for name, (_, cfg, w) in models.items()}


def check(got, ref, reqs, dtype):
    """float32: every position within the limit.  bfloat16: the rounding of a router's input can tip a choice between two
    experts whose scores are nearly equal, which changes that token (and, less, the later ones of its request) by more
    than rounding does elsewhere; so the typical position stays within the limit and few are far over it.  What is cut
    or placed wrongly shows in float32, where nothing is left to chance."""
    for rid, toks in reqs.items():
        assert sorted(got[rid]) == list(range(len(toks))), f"{rid}: positions missing"
        g = np.stack([got[rid][p] for p in range(len(toks))])
        assert np.isfinite(g).all(), f"{rid}: position {int((~np.isfinite(g)).any(axis=1).argmax())} is not finite"
        diff = g - ref[rid]
        err = (diff - diff.mean(axis=1, keepdims=True)).std(axis=1) / ref[rid].std()
        if dtype == "float32":
            assert err.max() <= F32_TOL, f"{rid}: first bad position {int((err > F32_TOL).argmax())}, worst {err.max():.2e}"
        else:
            over = err > 2 * BF16_TOL
            assert np.median(err) <= BF16_TOL and over.sum() <= max(1, len(toks) // 8), \
                f"{rid}: first bad position {int(over.argmax())}, {int(over.sum())} far over, median {np.median(err):.2e}"


def pairs(requests, n=2):
    return tt.portions(requests, sizes=(n,))


MODES = {"whole": tt.whole, "decode_tail": tt.decode_tail, "portions": tt.portions, "pairs": pairs, "mixed": tt.mixed}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("name", list(MODELS))
def test_replay_matches_plain(name, mode, dtype, models, references, tmp_path):
    folder, cfg, _ = models[name]
    reqs = requests_for(name)
    got = tt.run_trace(folder, dtype, MODES[mode](reqs), str(tmp_path), vocab=cfg["vocab"],
                       page_size=16 if name == "A" else 5)
    check(got, references[name], reqs, dtype)


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_logits_do_not_depend_on_the_cutting(name, models, tmp_path):
    """Every kernel fixes the order of its sums per output, so in float32 a position's logits are the same bits
    however its tokens were cut and batched, wherever its pages and its state slot lie, and whichever rows its
    choices got in the experts' ordering."""
    folder, cfg, _ = models[name]
    reqs = requests_for(name)
    outs = []
    for i, mode in enumerate(("whole", "portions", "mixed", "pairs")):
        d = tmp_path / mode
        d.mkdir()
        outs.append(tt.run_trace(folder, "float32", MODES[mode](reqs), str(d), page_size=(8, 16, 3, 64)[i]))
    for rid, toks in reqs.items():
        for p in range(len(toks)):
            for other in outs[1:]:
                assert np.array_equal(outs[0][rid][p], other[rid][p]), f"{rid} position {p} differs between cuttings"


def test_bfloat16_tensor_core_paths_agree_with_float32(models, tmp_path):
    """Pages of 64 keys and heads of 64 elements: in bfloat16 the last layer's prompt portions run in the tcgen05 kernel
    and its single tokens in the kernel that streams the cache by TMA, both with the chunk bound; the experts' products
    run on the tensor cores.  The same trace in float32 (CUDA cores throughout) is the comparison."""
    folder, cfg, _ = models["A"]
    reqs = {k: v for k, v in requests_for("A").items() if len(v) > 30}
    steps = tt.mixed(reqs, live=3, first=40)
    out = {}
    for dtype in ("float32", "bfloat16"):
        d = tmp_path / dtype
        d.mkdir()
        out[dtype] = tt.run_trace(folder, dtype, steps, str(d), vocab=cfg["vocab"], page_size=64)
    ref = {rid: np.stack([out["float32"][rid][p] for p in range(len(t))]) for rid, t in reqs.items()}
    check(out["bfloat16"], ref, reqs, "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_one_token(dtype, models, tmp_path):
    """One token of prompt, then 200 tokens one by one: state and cache written by single-token steps only, over many
    chunk borders (chunks of 24 and of 7) and page borders."""
    folder, cfg, w = models["A"]
    toks = np.random.default_rng(3).integers(0, cfg["vocab"], 201).tolist()
    reqs = {"long": toks}
    got = tt.run_trace(folder, dtype, tt.decode_tail(reqs, tail=200), str(tmp_path), vocab=cfg["vocab"], page_size=16)
    check(got, {"long": pn.forward(cfg, w, toks).numpy()}, reqs, dtype)


def plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(pn.forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("eager", [True, False])
def test_greedy_generation_through_the_engine(eager, name, models):
    """``LLM.generate`` with more prompts than state slots and a token budget that cuts prompts into portions: the
    scheduler admits, batches, frees and reuses pages and slots; tokens equal the plain model's greedy choice.  With
    captured decode steps (eager False) the experts' ordering is made on the device inside the captured step, and
    the batch is padded with idle entries that hold no slot."""
    from nanohybrid_vlm_b200 import LLM, SamplingParams
    folder, cfg, w = models[name]
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (23, 5, 41, 1, 12)]
    llm = LLM(folder, dtype="float32", kvcache_block_size=8, num_kvcache_blocks=40, max_num_batched_tokens=16,
              max_num_seqs=3, max_model_len=64, enforce_eager=eager)
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=7, ignore_eos=True), use_tqdm=False)
    for p, o in zip(prompts, out):
        assert o["token_ids"] == plain_greedy(cfg, w, p, 7)


def test_command_line_generates_the_plain_models_tokens(models):
    """``python -m nanohybrid_vlm_b200.cli generate`` on a Nomudra folder: the registry picks the model by config.json."""
    import subprocess
    import sys
    folder, cfg, w = models["B"]
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (6, 19)]
    args = [sys.executable, "-m", "nanohybrid_vlm_b200.cli", "generate", "--model", folder, "--dtype", "float32",
            "--temperature", "0", "--max-tokens", "5", "--ignore-eos", "--kvcache-block-size", "16", "--num-kvcache-blocks",
            "16", "--max-num-seqs", "2", "--max-model-len", "64", "--max-num-batched-tokens", "32", "--quiet"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    env = dict(os.environ, PYTHONPATH=tt.ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run(args, capture_output=True, text=True, env=env, cwd=tt.ROOT)
    assert r.returncode == 0, r.stderr[-3000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [l["token_ids"] for l in lines] == [plain_greedy(cfg, w, p, 5) for p in prompts]


def test_random_weights_folder_round_trip(tmp_path):
    """The random-weights mode writes a Nomudra folder from its configuration that the engine loads and runs."""
    from nanohybrid_vlm_b200.weights import write_random_model
    folder = str(tmp_path / "m")
    write_random_model(folder, dict(NOM_B, dtype="bfloat16"), seed=5)
    reqs = {"a": list(range(40)), "b": [7, 3, 9]}
    out = tmp_path / "o"
    out.mkdir()
    got = tt.run_trace(folder, "bfloat16", tt.mixed(reqs, live=2, first=8), str(out), vocab=NOM_B["vocab"])
    assert all(np.isfinite(row).all() for rows in got.values() for row in rows.values())
