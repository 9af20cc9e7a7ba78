"""The reference's own GPU worker on the B200, run unmodified, as (1) the pin of the CPU restatement and (2) the
proof that the kernel-entry image is a drop-in.

oracle/_ref/gpt2_infer is helixc/runtime/gpt2_infer.c compiled from the reference tree (oracle/Makefile, target
`ref`); oracle/_ref/kovc/*.ptx are the reference's kernels, emitted from its own kernel sources by its own compiler
(oracle/mint_ref_ptx.py).  Both are built where the reference tree is available and travel with the repository's
build outputs; the tests skip when they are absent.

  * worker + its own PTX, `--logits`: the unfused prefill of forward_full (gpt2_infer.c:1297-1333) on the GPU.  Its
    last-row logits are compared with the CPU restatement's (orc_model_prefill) -> the restatement's model-level
    sequencing is pinned by the reference itself.  The worker applies its own 5e-2 bar to the same pair
    (GPT2_LOGITS_PARITY_PASS, :2950-2954).
  * worker + its own PTX, `--generate` with the resident fused decode path (HX_KV HX_FAST HX_PACKEDRES HX_FUSEDGEMV
    HX_GEMV3 HX_FUSEDATTN, decode_step_llama :1341-1613): greedy tokens equal to orc_model_generate's.
  * the same two commands with helix_b200_kernels.fatbin given wherever the worker takes a PTX file: the reference's
    launcher (cuModuleLoadData / cuModuleGetFunction / cuLaunchKernel with its own grids) drives this library's
    kernels and reaches the same verdicts.
  * this library's decode engine on the same file against the worker's logits directly.

Shapes obey the worker's own limits: head_dim a multiple of 64 and every width a multiple of 64 (its tiled GEMM has
no edge handling, gpt2_infer.c:376-387); its KV decode path needs n_heads * head_dim == d_model (:1492-1504).
"""
import os
import subprocess

import numpy as np
import pytest

import helix_b200 as hb
import oracle_lib as ol

pytestmark = pytest.mark.gpu

KOVC = os.path.join(ol.ORACLE_DIR, "_ref", "kovc")
SIDE = dict(HX_DQPTX="nvfp4_dequant_tiled", HX_FUSEDGEMV_PTX="dequant_gemv_blockred", HX_GEMV3_PTX="dequant_gemv_warp",
            HX_FUSEDATTN_PTX="fused_decode_attn", HX_SPEC_PTX="softmax_causal_offset")
FUSED = dict(HX_KV="1", HX_FAST="1", HX_PACKEDRES="1", HX_FUSEDGEMV="1", HX_GEMV3="1", HX_FUSEDATTN="1")

CFGS = {
    "d256-gqa2-dh64": dict(NL=2, DM=256, NH=4, NKV=2, DH=64, DFF=512, NV=1000),
    "d512-gqa4-dh128": dict(NL=3, DM=512, NH=4, NKV=1, DH=128, DFF=768, NV=2011),
    "d256-qd512-dh128": dict(NL=2, DM=256, NH=4, NKV=2, DH=128, DFF=640, NV=1500),     # q width != d_model (the 32B geometry)
}
SEED_W, SEED_IDS, N_PROMPT, N_GEN = 41, 43, 11, 9


def have_worker():
    return os.path.exists(ol.REF_INFER) and os.path.exists(os.path.join(KOVC, "model14.ptx"))


def run_worker(image, weights, args, extra_env, cwd):
    """image: 'kovc' (the reference's own PTX) or 'ours' (this library's kernel image in every slot)."""
    env = {k: v for k, v in os.environ.items() if not k.startswith("HX_")}
    env.pop("LD_LIBRARY_PATH", None)
    if image == "kovc":
        main = os.path.join(KOVC, "model14.ptx")
        env.update({k: os.path.join(KOVC, v + ".ptx") for k, v in SIDE.items()})
    else:
        main = hb.fatbin_path()
        env.update({k: hb.fatbin_path() for k in SIDE})
    env.update(extra_env)
    p = subprocess.run([ol.REF_INFER, main, weights] + args, env=env, cwd=cwd, capture_output=True, text=True, timeout=600)
    return p.returncode, p.stdout + p.stderr


@pytest.fixture(scope="module", params=sorted(CFGS))
def case(request, tmp_path_factory):
    if not have_worker():
        pytest.skip("oracle/_ref/gpt2_infer or oracle/_ref/kovc/model14.ptx not built")
    cfg = CFGS[request.param]
    d = tmp_path_factory.mktemp("refw_" + request.param)
    path = str(d / "m.weights")
    ol.write_v3(path, cfg, ol.synth_tensors(cfg, seed=SEED_W))
    ids = np.random.default_rng(SEED_IDS).integers(0, cfg["NV"], N_PROMPT).astype(np.int32)
    open(d / "ids.txt", "w").write(" ".join(str(int(t)) for t in ids) + "\n")
    om = ol.OracleModel(path, kv_cap=64)
    lo = om.prefill(ids)
    gen = om.generate(ids, N_GEN)
    om.close()
    lo.tofile(d / "oracle_logits.bin")
    open(d / "oracle_argmax.txt", "w").write(f"{int(np.argmax(lo))}\n")
    open(d / "oracle_gen.txt", "w").write(" ".join(str(int(t)) for t in list(ids) + list(gen)) + "\n")
    return dict(name=request.param, cfg=cfg, dir=str(d), path=path, ids=ids, logits=lo, gen=gen)


@pytest.mark.parametrize("image", ["kovc", "ours"])
def test_worker_prefill_logits_against_the_cpu_restatement(case, image):
    d = case["dir"]
    rc, out = run_worker(image, case["path"], ["--logits", d + "/oracle_logits.bin", d + "/oracle_argmax.txt", d + "/ids.txt"],
                         dict(HX_FAST="1"), d)
    assert "GPT2_LOGITS_PARITY_PASS" in out and rc == 0, out[-3000:]
    got = np.fromfile("/tmp/helix_logits_last.bin", np.float32)
    err = float(np.max(np.abs(got - case["logits"])))
    print(f"{case['name']} [{image}] worker prefill vs CPU restatement: logits max-abs {err:.3g}")
    assert err < 2e-4                                   # observed ~1e-6; the worker's own bar is 5e-2
    if image == "kovc":
        # this library's engine against the reference GPU worker itself
        gm = hb.Model.load(case["path"], kv_cap=64)
        nx, lg = gm.prefill(case["ids"], want_logits=True)
        gm.close()
        assert float(np.max(np.abs(lg - got))) < 2e-4 and nx == int(np.argmax(got))
        out_dir = os.environ.get("HX_REF_WORKER_DUMP")
        if out_dir:                                      # fixture capture for tests/golden (make_ref_worker_golden.py)
            np.save(os.path.join(out_dir, f"ref_worker_logits_{case['name']}.npy"), got)


@pytest.mark.parametrize("image", ["kovc", "ours"])
def test_worker_fused_decode_tokens_against_the_cpu_restatement(case, image):
    if case["cfg"]["NH"] * case["cfg"]["DH"] != case["cfg"]["DM"]:
        pytest.skip("the worker's KV decode path needs n_heads * head_dim == d_model")
    d = case["dir"]
    rc, out = run_worker(image, case["path"], ["--generate", str(N_GEN), d + "/ids.txt", d + "/oracle_gen.txt"], FUSED, d)
    assert "TOKEN_FOR_TOKEN_MATCH" in out and "GPT2_GENERATE_MATCH_PASS" in out and rc == 0, out[-3000:]
    assert "fused dequant-GEMV module ON" in out and "HX_GEMV3 ACTIVE" in out, out[-3000:]


N_SPEC = 48


@pytest.mark.parametrize("image", ["kovc", "ours"])
def test_worker_speculative_decode_against_this_library(case, image):
    """The worker's HX_SPEC path (pld_draft / forward_verify / spec_step, gpt2_infer.c:2972-3118) on a prompt that
    repeats: its tokens are the plain greedy tokens, and its [specprof] counters equal both the token-level replay of
    its accept rule (oracle_lib.spec_counters) and the counters of hx_generate_spec on the same file."""
    import re
    if case["cfg"]["NH"] * case["cfg"]["DH"] != case["cfg"]["DM"]:
        pytest.skip("the worker's KV decode path needs n_heads * head_dim == d_model")
    d = case["dir"]
    base = np.random.default_rng(SEED_IDS + 1).integers(0, case["cfg"]["NV"], 5).astype(np.int32)
    prompt = np.concatenate([base, base, base[:3]]).astype(np.int32)
    om = ol.OracleModel(case["path"], kv_cap=128)
    greedy = om.generate(prompt, N_SPEC)
    om.close()
    open(d + "/ids_spec.txt", "w").write(" ".join(str(int(t)) for t in prompt) + "\n")
    open(d + "/oracle_gen_spec.txt", "w").write(" ".join(str(int(t)) for t in list(prompt) + list(greedy)) + "\n")
    rc, out = run_worker(image, case["path"], ["--generate", str(N_SPEC), d + "/ids_spec.txt", d + "/oracle_gen_spec.txt"],
                         dict(HX_KV="1", HX_FAST="1", HX_SPEC="1"), d)
    assert "TOKEN_FOR_TOKEN_MATCH" in out and rc == 0, out[-3000:]
    mt = re.search(r"\[specprof\] steps=(\d+) hits=(\d+) drafted=(\d+) accepted=(\d+) emitted=(\d+) forwards=(\d+)", out)
    assert mt, out[-3000:]
    worker = dict(zip(ol.SPEC_COUNTERS, [int(v) for v in mt.groups()]))
    replay = ol.spec_counters(prompt, greedy)
    print(f"{case['name']} [{image}] worker specprof {worker}")
    assert worker == replay
    assert worker["accepted"] > 0                        # the toy models repeat themselves: drafts are accepted
    gm = hb.Model.load(case["path"], kv_cap=128)
    spec, st, _, _ = gm.generate_spec(prompt, N_SPEC)
    gm.close()
    assert list(spec) == list(greedy)
    if st["near_ties"] == 0:
        assert {k: st[k] for k in ol.SPEC_COUNTERS} == worker
