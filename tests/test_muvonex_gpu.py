"""Muvonex through the engine against the plain model (float64, token by token): the same requests whole, with
their last tokens decoded one by one, in portions down to two tokens, and mixed with other requests in a pool so
small that pages and state slots are used again; long decoding from a single token; greedy generation through
``LLM.generate`` and the scheduler.  Small configurations that differ in every size, in the order of their
layers and in every option: groups of several heads, norm groups, a layer without a feed-forward, rotation of a
part of the head, frequency bands or none, one tap and many; one without attention, one whose attention has key
and value heads of one size."""
import json
import os

import numpy as np
import pytest
import torch

import plain_muvonex as pm
import trace_tools as tt

pytestmark = pytest.mark.gpu


def delta(heads, kv, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv)


def parallel(left, right, ls, rs):
    return dict(left=left, right=right, left_scale=ls, right_scale=rs)


MUV_A = dict(
    architecture="Muvonex", vocab=320, width=128, embedding=dict(scale=8.0), norm=dict(eps=1e-5), residual_mult=0.5,
    layers=[
        dict(type="parallel", mlp=dict(kind="dense", ff=192), mixer=parallel(
            dict(heads=4, kv_heads=1, dim=64, vdim=32, scale=0.2, rot=dict(base=10000.0, dims=32, scaling=None)),
            dict(heads=4, groups=2, state=16, vdim=24, conv=3, norm_groups=2), 1.3, 0.6)),
        dict(type="delta", mlp=None, mixer=delta(4, 2, 24, 40, 2)),
        dict(type="parallel", mlp=dict(kind="dense", ff=64), mixer=parallel(
            dict(heads=2, kv_heads=2, dim=16, vdim=48, scale=0.5, rot=dict(base=500.0, dims=16, scaling=dict(
                factor=8.0, low=1.0, high=4.0, original=64))),
            dict(heads=3, groups=1, state=40, vdim=36, conv=1, norm_groups=3), 0.7, 1.0)),
    ])
MUV_B = dict(
    architecture="Muvonex", vocab=501, width=192, embedding=dict(scale=3.0), norm=dict(eps=1e-6), residual_mult=1.0,
    layers=[
        dict(type="delta", mlp=dict(kind="dense", ff=200), mixer=delta(3, 3, 48, 32, 5)),
        dict(type="delta", mlp=dict(kind="dense", ff=100), mixer=delta(2, 1, 72, 72, 4)),
        dict(type="parallel", mlp=None, mixer=parallel(
            dict(heads=8, kv_heads=4, dim=40, vdim=72, scale=0.16, rot=dict(base=250000.0, dims=20, scaling=dict(
                factor=4.0, low=1.0, high=4.0, original=32))),
            dict(heads=6, groups=3, state=24, vdim=20, conv=4, norm_groups=1), 1.0, 1.0)),
        dict(type="delta", mlp=dict(kind="dense", ff=64), mixer=delta(5, 1, 32, 40, 1)),
    ])
# no attention anywhere: nothing is kept in pages, only state slots; sizes that are no multiple of 4
MUV_C = dict(
    architecture="Muvonex", vocab=97, width=72, embedding=dict(scale=1.0), norm=dict(eps=1e-6), residual_mult=0.7,
    layers=[
        dict(type="delta", mlp=dict(kind="dense", ff=90), mixer=delta(2, 2, 34, 38, 3)),
        dict(type="delta", mlp=None, mixer=delta(6, 3, 32, 48, 8)),
    ])
# key and value heads of one size, in steps of 16: in bfloat16 this attention runs on the tensor cores
MUV_D = dict(
    architecture="Muvonex", vocab=260, width=96, embedding=dict(scale=4.0), norm=dict(eps=1e-6), residual_mult=0.4,
    layers=[
        dict(type="parallel", mlp=dict(kind="dense", ff=128), mixer=parallel(
            dict(heads=6, kv_heads=2, dim=48, vdim=48, scale=0.15, rot=dict(base=10000.0, dims=48, scaling=dict(
                factor=2.0, low=1.0, high=2.0, original=24))),
            dict(heads=2, groups=1, state=32, vdim=48, conv=4, norm_groups=1), 0.9, 1.2)),
        dict(type="delta", mlp=dict(kind="dense", ff=128), mixer=delta(3, 3, 32, 32, 4)),
        dict(type="parallel", mlp=None, mixer=parallel(
            dict(heads=2, kv_heads=1, dim=64, vdim=64, scale=0.125, rot=dict(base=10000.0, dims=32, scaling=None)),
            dict(heads=4, groups=2, state=16, vdim=32, conv=2, norm_groups=2), 1.0, 1.0)),
    ])
MODELS = {"A": (MUV_A, 11), "B": (MUV_B, 12), "C": (MUV_C, 13), "D": (MUV_D, 14)}
LENGTHS = (70, 41, 97, 2, 33, 129, 1, 9, 55)
# the root mean square over the vocabulary of a position's error (its mean taken off: a shift of all logits changes
# no probability), as a share of the spread of the logits
F32_TOL = 1e-4          # float32 sums in another order than float64
BF16_TOL = 0.05         # activations rounded to 8 bits of mantissa after every op


def write_model(folder, cfg, seed):
    from safetensors.torch import save_file
    w = pm.random_weights(cfg, seed)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(folder, "model.safetensors"))
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return {k: v.to(torch.float64) for k, v in w.items()}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, seed) in MODELS.items():
        d = str(tmp_path_factory.mktemp(f"muvonex_{name}"))
        out[name] = (d, cfg, write_model(d, cfg, seed))
    return out


def requests_for(name):
    cfg, seed = MODELS[name]
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(LENGTHS)}


@pytest.fixture(scope="module")
def references(models):
    return {name: {rid: pm.forward(cfg, w, t).numpy() for rid, t in requests_for(name).items()}
            for name, (_, cfg, w) in models.items()}


def check(got, ref, reqs, dtype):
    limit = F32_TOL if dtype == "float32" else BF16_TOL
    for rid, toks in reqs.items():
        assert sorted(got[rid]) == list(range(len(toks))), f"{rid}: positions missing"
        g = np.stack([got[rid][p] for p in range(len(toks))])
        assert np.isfinite(g).all(), f"{rid}: position {int((~np.isfinite(g)).any(axis=1).argmax())} is not finite"
        diff = g - ref[rid]
        err = (diff - diff.mean(axis=1, keepdims=True)).std(axis=1) / ref[rid].std()
        # bfloat16: a position where a norm divides by a root mean square that happens to be small multiplies the
        # rounding of its inputs; such a position may reach twice the limit, the others stay under it
        over = err > limit
        assert err.max() <= (1.0 if dtype == "float32" else 2.0) * limit and over.sum() <= len(toks) // 50, \
            f"{rid}: first bad position {int(over.argmax())}, {int(over.sum())} over, worst {err.max():.2e} of the spread"


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
    however its tokens were cut and batched, and wherever its pages and its state slot lie."""
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_one_token(dtype, models, tmp_path):
    """One token of prompt, then 180 tokens one by one: state and cache written by single-token steps only."""
    folder, cfg, w = models["A"]
    toks = np.random.default_rng(3).integers(0, cfg["vocab"], 181).tolist()
    reqs = {"long": toks}
    got = tt.run_trace(folder, dtype, tt.decode_tail(reqs, tail=180), str(tmp_path), vocab=cfg["vocab"], page_size=16)
    check(got, {"long": pm.forward(cfg, w, toks).numpy()}, reqs, dtype)


def plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(pm.forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["B", "C"])
@pytest.mark.parametrize("eager", [True, False])
def test_greedy_generation_through_the_engine(eager, name, models):
    """``LLM.generate`` with more prompts than state slots and a token budget that cuts prompts into portions: the
    scheduler admits, batches, frees and reuses slots; tokens equal the plain model's greedy choice.  With captured
    decode steps (eager False) the batch is padded with idle entries that hold no slot."""
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
    """``python -m nanohybrid_vlm_b200.cli generate`` on a Muvonex folder: the registry picks the model by config.json."""
    import subprocess
    import sys
    folder, cfg, w = models["A"]
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
