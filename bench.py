#!/usr/bin/env python
"""Benchmark of the NVFP4 decode path: greedy batch-1 decode of a Qwen3-8B-shaped model with seeded
synthetic weights, 512-token prompt, 256 new tokens.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one 256-token greedy continuation from position 512 of the prompt's KV cache.  `value`
is decoded tokens per second with everything resident in HBM (CUDA events around the K steps, max over
ranks); `e2e` is the same metric through the public per-token call hx_decode_step with host buffers
(token id in, next id and the logits row out, every token).  With N > 1 each GPU holds a full weight
copy and decodes its own sequence (independent sequences, no data-path collective): weak scaling.

Beside the headline the line carries
  parity         logits and greedy tokens of the GPU path against the CPU restatement on the same weights
  reference_gpu  the reference's own worker (its C host program + its own compiler's PTX) on this GPU, same model
                 shape at reduced depth, next to this library at that depth
  batch64        64 independent sequences, 2048-token prompts + 128 decoded tokens each, split over the GPUs
  tp             the Qwen3-32B shape as ONE tensor-parallel group over the N GPUs (N = 1: one GPU)
  quantizer, gpt2, prefill, batched_decode   the other configurations of the path.

`--impl reference` times the CPU restatement of the reference worker's decode (oracle/hx_oracle.c, all
host threads) on the same model shape; rank 0 alone runs it.
"""
import argparse
import ctypes as C
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_LEN, NEW_TOKENS = 512, 256
BATCH_SEQS, BATCH_PROMPT, BATCH_NEW = 64, 2048, 128      # the batched-throughput configuration
TP_PROMPT, TP_NEW = 4096, 64                             # 32B shape: context length, decoded tokens timed
TP_BATCH, TP_BATCH_STEPS = 16, 16                        # 32B shape: sequences decoded together inside the group, steps timed
# DRAM bytes / algorithmic bytes of the decode kernel, from one ncu capture of a 4-layer launch (see the summary
# kept with the ncu summaries of that kernel); re-measured when the kernel's memory traffic changes
NCU_TRAFFIC_RATIO = 1.012
WORKLOAD = "qwen3-8b-shape nvfp4 greedy decode, batch 1, 512-token prompt + 256 new tokens"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, dev):
        self.dev, self.proc, self.lines = dev, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.dev), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_init(n):
    if n <= 1:
        return None
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
    return dist


def all_max(dist, v):
    if dist is None:
        return v
    import torch
    t = torch.tensor([v], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def all_sum(dist, v):
    if dist is None:
        return v
    import torch
    t = torch.tensor([v], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t[0])


def algorithmic_bytes_per_token(cfg, T):
    """0.5625 B per logical weight of every linear incl. lm_head + the fp32 KV rows read + one embedding row."""
    NL, DM, NH, NKV, DH, DFF, NV = (cfg[k] for k in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "d_ff", "vocab"))
    QD, KVD = NH * DH, NKV * DH
    weights = NL * (QD * DM + 2 * KVD * DM + DM * QD + 2 * DFF * DM + DM * DFF) + NV * DM
    return weights * 0.5625, 2 * NL * NKV * DH * 4 * T, DM * 4


def synth_image_on_host(shape, seed):
    """An HXGW v3 image of the given shape built on the host without the GPU: codes and scale bytes are
    drawn directly in the committed layout (uniform codes, scale bytes in the range the quantizer emits
    for N(0, 0.02) weights).  It costs the CPU decode exactly what a quantized checkpoint costs."""
    import struct
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    cfg = dict(NL=shape["n_layers"], DM=shape["d_model"], NH=shape["n_heads"], NKV=shape["n_kv_heads"], DH=shape["head_dim"],
               DFF=shape["d_ff"], NV=shape["vocab"])
    order = ol.qwen3_tensor_order(cfg)
    rng = np.random.default_rng(seed)
    sizes, cur = [], 64 + 32 * len(order)
    for name, shp, packed in order:
        if packed:
            kp = ol.kpad(shp[1]); n = shp[0] * (kp // 7) * 4 + shp[0] * (kp // 16) + 4
        else:
            n = int(np.prod(shp)) * 4
        sizes.append(n); cur += n
    img = np.empty(cur, np.uint8)
    hdr = bytearray(64)
    struct.pack_into("<8I", hdr, 0, 0x48584757, 3, cfg["NL"], cfg["DM"], cfg["NH"], cfg["NV"], 40960, cfg["DFF"])
    struct.pack_into("<II", hdr, 40, 1, cfg["NKV"]); struct.pack_into("<ff", hdr, 48, 1e6, 1e-6)
    struct.pack_into("<II", hdr, 56, cfg["DH"], len(order))
    img[:64] = np.frombuffer(bytes(hdr), np.uint8)
    off, dpos = 64 + 32 * len(order), 64
    for (name, shp, packed), n in zip(order, sizes):
        if packed:
            rows, K = shp; kp = ol.kpad(K); wb = rows * (kp // 7) * 4; mb = rows * (kp // 16)
            img[dpos:dpos + 32] = np.frombuffer(struct.pack("<IIIIQQ", 1, rows, K, kp, off, off + wb), np.uint8)
            img[off:off + wb] = rng.integers(0, 256, wb, dtype=np.uint8)
            img[off + 3:off + wb:4] &= 0x0F                       # 28-bit words: the top nibble is empty
            img[off + wb:off + wb + mb] = rng.integers(0x28, 0x7F, mb, dtype=np.uint8)
            img[off + wb + mb:off + n] = np.frombuffer(struct.pack("<f", 4.2e-5), np.uint8)
        else:
            cnt = int(np.prod(shp))
            img[dpos:dpos + 32] = np.frombuffer(struct.pack("<IIIIQQ", 0, 1, cnt, cnt, off, 0), np.uint8)
            v = img[off:off + n].view(np.float32)
            if len(shp) == 1:
                v[:] = 1.0
            else:
                step = 1 << 24
                for s in range(0, cnt, step):
                    e = min(cnt, s + step)
                    v[s:e] = rng.standard_normal(e - s, dtype=np.float32) * np.float32(0.02)
        off += n; dpos += 32
    return img


def oracle_lib_all_cores():
    if "oracle_lib" not in sys.modules:
        # all host cores, also under torchrun (which exports OMP_NUM_THREADS=1); read when the OpenMP runtime starts
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    return ol


def cpu_decode_tok_s(image, n_tokens, kv_cap=64):
    """tokens/s of the CPU restatement decoding n_tokens greedy tokens from an empty cache."""
    ol = oracle_lib_all_cores()
    om = ol.OracleModel(image=image, kv_cap=kv_cap)
    tok, t0 = 1, time.perf_counter()
    for pos in range(n_tokens):
        tok = int(np.argmax(om.decode(tok, pos)))
    dt = time.perf_counter() - t0
    om.close()
    return n_tokens / dt, ol.oracle().orc_num_threads()


def cpu_baseline_with_parity(model, budget_s=20.0):
    """The CPU restatement on the SAME weights (HXGW v3 image exported from HBM), teacher-forced along the GPU's
    own greedy tokens from an empty cache: tokens/s of the CPU leg and, position by position, the logits and
    arg-max of both sides."""
    ol = oracle_lib_all_cores()
    image = model.v3_image()
    om = ol.OracleModel(image=image, kv_cap=64)
    gpu_tok, cpu_free, max_abs, frel, agree_tf, cpu_s = [1], 1, 0.0, 0.0, 0, 0.0
    n, pos, free_ok, free_agree = 2, 0, True, 0
    while pos < n:
        tok = gpu_tok[pos]
        nx, lg = model.decode_step(tok, pos, want_logits=True)
        t0 = time.perf_counter()
        lo = om.decode(tok, pos)
        dt = time.perf_counter() - t0
        cpu_s += dt
        if pos == 0:
            n = int(max(2, min(16, budget_s / dt)))
        d = np.abs(lg - lo)
        max_abs = max(max_abs, float(d.max()))
        frel = max(frel, float(np.max(d / np.maximum(np.abs(lo), 1.0))))
        ca = int(np.argmax(lo))
        agree_tf += int(ca == nx)
        # free-running: the CPU would have fed its own arg-max; the runs coincide as long as every earlier one agreed
        free_ok = free_ok and ca == nx
        free_agree += int(free_ok)
        gpu_tok.append(nx)
        pos += 1
    om.close()
    cores = ol.oracle().orc_num_threads()
    cpu = {"value": n / cpu_s, "unit": "tok/s", "cores": cores, "kind": "port",
           "sample": f"{n} tokens from an empty KV cache on the same weights (HXGW v3 image exported from the GPU), full "
                     "model + lm_head, teacher-forced along the GPU's greedy tokens; CPU restatement of the reference "
                     "decode, OpenMP over rows"}
    parity = {"tokens": n, "logit_max_abs": max_abs, "floored_rel": frel,
              "greedy_agree_teacher_forced": agree_tf / n, "greedy_agree_free": free_agree / n,
              "bars": "reference: max-abs < 5e-2, |d| / max(|ref|, 1) < 1e-3, arg-max equal",
              "against": "CPU restatement, itself pinned by the reference's GPU worker (tests/golden/ref_worker_logits.npz)"}
    del image
    return cpu, parity


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)    # torchrun exports 1; the CPU arm uses every host core
    import helix_b200 as hb
    shape = dict(hb.QWEN3_8B)
    image = synth_image_on_host(shape, seed=1)
    n_tok = 2
    for _ in range(args.warmup):
        cpu_decode_tok_s(image, 1)
    t0 = time.perf_counter()
    vals = []
    cores = 1
    for _ in range(args.steps):
        v, cores = cpu_decode_tok_s(image, n_tok)
        vals.append(v)
    wall = time.perf_counter() - t0
    value = args.steps * n_tok / sum(n_tok / v for v in vals)
    sample = f"{n_tok} greedy tokens per step from an empty KV cache (positions 0..{n_tok - 1}), full 36-layer model + lm_head"
    line = {"metric": "nvfp4_decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": {"workload": WORKLOAD, "reference_arm": "CPU restatement of the reference decode (oracle/hx_oracle.c); "
                       "the reference's own CPU build covers GPT-2 f32 only"},
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def reference_gpu_leg(hb, layers, n_prompt=16, n_gen=24):
    """The reference's own GPU path on this GPU: its worker (helixc/runtime/gpt2_infer.c compiled unmodified) driving
    the PTX its own compiler emits, resident fused decode path, on an HXGW v3 file this library exports -- beside this
    library on the same file.  Depth is reduced so that the file (the f32 embedding alone is 2.5 GB) is written and
    loaded within seconds; widths, vocabulary and per-layer work are the benchmark's."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    kovc = os.path.join(ol.ORACLE_DIR, "_ref", "kovc")
    if not (os.path.exists(ol.REF_INFER) and os.path.exists(os.path.join(kovc, "model14.ptx"))):
        return {"unavailable": "oracle/_ref/gpt2_infer or oracle/_ref/kovc/*.ptx not built (make -C oracle ref)"}
    shape = dict(hb.QWEN3_8B); shape["n_layers"] = layers
    model = hb.Model.synth(shape, seed=1, kv_cap=n_prompt + n_gen + 8, flags=hb.HX_LOAD_KEEP_COMMITTED)
    prompt = np.random.default_rng(4).integers(0, shape["vocab"], n_prompt).astype(np.int32)
    model.generate(prompt, 4)
    ours, ms_p, ms_d = model.generate(prompt, n_gen)
    out = {"layers": layers, "prompt": n_prompt, "new_tokens": n_gen, "ours_ms_per_token": ms_d / (n_gen - 1),
           "engine": model.engine()}
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.weights")
        model.save_v3(path)
        model.close()
        open(os.path.join(d, "ids.txt"), "w").write(" ".join(str(int(t)) for t in prompt) + "\n")
        env = {k: v for k, v in os.environ.items() if not k.startswith("HX_")}
        env.update(HX_KV="1", HX_FAST="1", HX_PACKEDRES="1", HX_FUSEDGEMV="1", HX_GEMV3="1", HX_FUSEDATTN="1", HX_GENPROF="1",
                   HX_DQPTX=os.path.join(kovc, "nvfp4_dequant_tiled.ptx"), HX_FUSEDGEMV_PTX=os.path.join(kovc, "dequant_gemv_blockred.ptx"),
                   HX_GEMV3_PTX=os.path.join(kovc, "dequant_gemv_warp.ptx"), HX_FUSEDATTN_PTX=os.path.join(kovc, "fused_decode_attn.ptx"))
        t0 = time.perf_counter()
        try:
            p = subprocess.run([ol.REF_INFER, os.path.join(kovc, "model14.ptx"), path, "--generate", str(n_gen), os.path.join(d, "ids.txt")],
                               env=env, cwd=d, capture_output=True, text=True, timeout=240)
        except subprocess.TimeoutExpired:
            return dict(out, unavailable="the reference worker did not finish within 240 s")
        out["worker_wall_s"] = time.perf_counter() - t0
    txt = p.stdout + p.stderr
    m = re.search(r"\[genprof\] decode (\d+) steps in ([0-9.]+)s = ([0-9.]+) s/tok", txt)
    g = re.search(r"HELIX_GEN_IDS:((?: \d+)+)", txt)
    if p.returncode != 0 or not m or not g:
        return dict(out, unavailable="the reference worker failed: " + txt[-300:].replace("\n", " | "))
    ref_ids = [int(x) for x in g.group(1).split()][n_prompt:]
    out.update(reference_ms_per_token=float(m.group(3)) * 1e3, reference_decode_steps=int(m.group(1)),
               tokens_identical=ref_ids == [int(t) for t in ours],
               ratio=float(m.group(3)) * 1e3 / (ms_d / (n_gen - 1)),
               path="gpt2_infer.c + kovc PTX (sm_86 PTX JIT-compiled by the driver), HX_KV HX_FAST HX_PACKEDRES HX_FUSEDGEMV "
                    "HX_GEMV3 HX_FUSEDATTN, timed by its own HX_GENPROF")
    return out


def batch64_leg(hb, L, check, dist, rank, ngpus, shape):
    """64 independent sequences, each a 2048-token prompt then 128 greedy tokens, split over the GPUs; every GPU
    holds its own weight copy, prefills its sequences into their KV slots and decodes them together."""
    S = max(1, BATCH_SEQS // ngpus)
    model = hb.Model.synth(shape, seed=1, kv_cap=BATCH_PROMPT + BATCH_NEW + 8, batch=S)
    rng = np.random.default_rng(100 + rank)
    prompts = rng.integers(0, shape["vocab"], (S, BATCH_PROMPT)).astype(np.int32)
    model.prefill_seq(0, prompts[0][:64])                     # warm-up: graph capture of a chunk, first launches
    check(L.hx_sync())
    t0 = time.perf_counter()
    first = np.zeros(S, np.int32)
    first[0] = model.prefill_seq(0, prompts[0])
    t_one = time.perf_counter() - t0
    # the whole job must stay within the benchmark's time budget: fewer sequences per GPU when one prompt is slow
    S_run = S if t_one * S < 80.0 else max(4, int(80.0 / t_one))
    for s in range(1, S_run):
        first[s] = model.prefill_seq(s, prompts[s])
    prefill_s = all_max(dist, time.perf_counter() - t0)
    model.decode_batch_loop(first[:S_run], BATCH_PROMPT, 2)
    _, dms = model.decode_batch_loop(first[:S_run], BATCH_PROMPT, BATCH_NEW - 1)
    dms = all_max(dist, dms)
    model.close()
    n_seq = S_run * ngpus
    ptok, dtok = n_seq * BATCH_PROMPT, n_seq * (BATCH_NEW - 1)
    return {"sequences": n_seq, "sequences_asked": BATCH_SEQS, "per_gpu": S_run, "prompt": BATCH_PROMPT, "new_tokens": BATCH_NEW,
            "prefill_s": prefill_s, "prefill_tok_per_s": ptok / prefill_s, "decode_s": dms * 1e-3, "decode_tok_per_s": dtok / (dms * 1e-3),
            "total_tok_per_s": (ptok + dtok) / (prefill_s + dms * 1e-3),
            "path": "hx_prefill_seq per sequence (64-token chunks through the tcgen05 GEMM), then hx_decode_batch_loop "
                    "(64 sequences per pass over the weights); replicas, no exchange between GPUs"}


def tp_leg(hb, L, check, dist, rank, ngpus, peak):
    """The Qwen3-32B shape as one tensor-parallel group over the GPUs of the run, batch 1: the 4096-token prompt is
    prefilled in chunks of 64 positions (the partial rows of o_proj / down_proj exchanged per chunk), then tokens are
    decoded at that context."""
    shape = dict(hb.QWEN3_32B)
    cap = TP_PROMPT + TP_NEW + 16
    if ngpus > 1:
        import torch
        model = hb.Model.synth(shape, seed=1, kv_cap=cap, tp_rank=rank, tp_size=ngpus, batch=TP_BATCH)
        mine = torch.tensor(list(model.tp_handle()), dtype=torch.uint8)
        allh = [torch.zeros(64, dtype=torch.uint8) for _ in range(ngpus)]
        dist.all_gather(allh, mine)
        model.tp_connect([bytes(h.tolist()) for h in allh])
        dist.barrier()
    else:
        model = hb.Model.synth(shape, seed=1, kv_cap=cap, batch=TP_BATCH)
    prompt = np.random.default_rng(17).integers(0, shape["vocab"], TP_PROMPT).astype(np.int32)
    model.prefill(prompt[:64])                        # warm-up of the chunk path
    model.reset()
    if dist is not None:
        dist.barrier()
    tp0 = time.perf_counter()
    first = model.prefill(prompt)
    pf_s = all_max(dist, time.perf_counter() - tp0)
    model.decode_loop(first, TP_PROMPT, 8)
    if dist is not None:
        dist.barrier()
    _, ms = model.decode_loop(first, TP_PROMPT, TP_NEW)
    ms = all_max(dist, ms)
    cfg = dict(shape)
    wbytes, kvb, emb = algorithmic_bytes_per_token(cfg, TP_PROMPT + TP_NEW // 2)
    per_gpu = (wbytes + kvb) / ngpus + emb
    ms_tok = ms / TP_NEW
    engine = model.engine()
    # sixteen sequences through the group at the same context (their cache rows seeded synthetically: sixteen 4096-token
    # prefills would take minutes), one token each per step: the batched GEMM path with the row-split linears' partial
    # rows and the per-sequence arg-max exchanged between the ranks
    model.fill_kv(TP_PROMPT, 13)
    ids16 = np.random.default_rng(19).integers(0, shape["vocab"], TP_BATCH).astype(np.int32)
    model.decode_batch_loop(ids16, TP_PROMPT, 2)
    if dist is not None:
        dist.barrier()
    _, ms16 = model.decode_batch_loop(ids16, TP_PROMPT, TP_BATCH_STEPS)
    ms16 = all_max(dist, ms16)
    batch16 = {"sequences": TP_BATCH, "steps": TP_BATCH_STEPS, "context": TP_PROMPT, "tok_per_s": TP_BATCH * TP_BATCH_STEPS / (ms16 * 1e-3),
               "ms_per_step": ms16 / TP_BATCH_STEPS, "kv": "synthetic rows", "path": "hx_decode_batch_loop inside the group"}
    model.close()
    return {"model": "qwen3-32b-shape", "tp": ngpus, "batch": 1, "context": TP_PROMPT, "new_tokens": TP_NEW,
            "prefill_s": pf_s, "prefill_tok_per_s": TP_PROMPT / pf_s, "tok_per_s": 1e3 / ms_tok,
            "ms_per_token": ms_tok, "per_gpu_bytes_per_token": per_gpu, "per_gpu_frac_of_hbm_peak": per_gpu / (ms_tok * 1e-3) / 1e9 / peak,
            "engine": engine, "batch16": batch16,
            "exchange": "partial rows of o_proj / down_proj stored as (value, epoch) pairs into every rank's buffer over NVLink "
                        "inside the decode kernel, summed in rank order; no NCCL kernel" if ngpus > 1 else "none (one GPU)"}


def run_ours(args):
    import helix_b200 as hb
    from helix_b200.lib import check, lib
    dist = dist_init(args.gpus)
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    L = lib()
    check(L.hx_set_device(local))
    shape = dict(hb.QWEN3_32B if args.model == "32b" else hb.QWEN3_8B)
    if args.layers:
        shape["n_layers"] = args.layers                 # reduced-depth case for profiler captures; not a bench line
    keep = 1 if (rank == 0 and args.gpus == 1 and not args.no_cpu_baseline) else 0
    tp = args.parallelism == "tp" and args.gpus > 1
    if tp:
        import torch
        model = hb.Model.synth(shape, seed=1, kv_cap=PROMPT_LEN + NEW_TOKENS + 8, tp_rank=rank, tp_size=args.gpus)
        mine = torch.tensor(list(model.tp_handle()), dtype=torch.uint8)
        allh = [torch.zeros(64, dtype=torch.uint8) for _ in range(args.gpus)]
        dist.all_gather(allh, mine)
        model.tp_connect([bytes(h.tolist()) for h in allh])
        dist.barrier()
    else:
        model = hb.Model.synth(shape, seed=1, kv_cap=PROMPT_LEN + NEW_TOKENS + 8, flags=keep)
    cfgd = model.cfg.as_dict()
    if tp:                                              # the shard reports its own slice; bytes are counted for the whole model
        for k in ("n_heads", "n_kv_heads", "d_ff", "vocab"):
            cfgd[k] = shape[k]
    rng = np.random.default_rng(2 + (0 if tp else rank))
    prompt = rng.integers(0, shape["vocab"], PROMPT_LEN).astype(np.int32)
    model.prefill(prompt[:32])                         # warm-up (graph capture, first launches)
    check(L.hx_sync())
    tp0 = time.perf_counter()
    first = model.prefill(prompt)                      # real KV for positions 0..511 + the first new token
    prefill_s = time.perf_counter() - tp0              # hx_prefill returns after the stream has drained
    dbytes, cbytes = model.weight_bytes()

    def one_step():
        return model.decode_loop(first, PROMPT_LEN, NEW_TOKENS)

    for _ in range(args.warmup):
        one_step()
    if dist is not None:
        dist.barrier()
    check(L.hx_sync())
    sampler = ClockSampler(local); sampler.start()
    l0 = hb.launch_count()
    ms_total, toks = 0.0, None
    for _ in range(args.steps):
        toks, ms = one_step()
        ms_total += ms
    check(L.hx_sync())
    launches = hb.launch_count() - l0
    clocks = sampler.stop()
    if dist is not None:
        dist.barrier()
    ms_max = all_max(dist, ms_total)
    n_seq = 1 if tp else args.gpus
    n_tok_all = n_seq * args.steps * NEW_TOKENS
    value = n_tok_all / (ms_max * 1e-3)

    wbytes, kvbytes_mid, embbytes = algorithmic_bytes_per_token(cfgd, PROMPT_LEN + NEW_TOKENS // 2)
    token_bytes = wbytes + kvbytes_mid + embbytes
    peak, peak_src = peaks()
    engine = model.engine()
    if engine.startswith("persistent"):
        # The whole token is ONE cooperative launch of the persistent kernel, so the dominant kernel's average
        # launch duration is the timed region (CUDA events on the launching stream inside hx_decode_loop) over
        # the launches in it, and its algorithmic bytes are the token's.
        n_launch = args.steps * NEW_TOKENS
        avg_ms = ms_total / n_launch
        achieved = token_bytes / (avg_ms * 1e-3) / 1e9
        kname = "k_decode_df" if engine.endswith("dataflow") else ("k_decode_tc" if engine.endswith("tcgen05") else "k_decode_persist")
        roofline = {"bound": "hbm", "kernel": f"{kname} (persistent cooperative kernel, one launch = one decoded token: all "
                    f"{4 * cfgd['n_layers'] + 1} linears, attention, norms, arg-max)",
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": token_bytes * NCU_TRAFFIC_RATIO if kname in ("k_decode_tc", "k_decode_df") else None,
                    "traffic_source": f"ncu dram__bytes_read+write of one launch of the 4-layer case = {NCU_TRAFFIC_RATIO} x its algorithmic "
                                      "bytes, scaled to this launch's algorithmic bytes (traffic grows with the layers streamed)",
                    "peak_source": peak_src, "algorithmic_bytes_per_launch": token_bytes, "avg_launch_us": avg_ms * 1e3,
                    "token_bytes": {"weights": wbytes, "kv_mid_run": kvbytes_mid, "embedding_row": embbytes},
                    "whole_token_frac": token_bytes * value / args.gpus / 1e9 / peak}
        if tp:      # every GPU streams 1/N of the weights and KV per launch
            roofline["algorithmic_bytes_per_launch"] = token_bytes / args.gpus
            roofline["achieved"] = achieved / args.gpus
            roofline["frac"] = achieved / args.gpus / peak
            roofline["traffic"] = None
    else:
        # per-kernel device time of the dominant kernel (k_linear), event pair around every launch
        model.set_profile(True)
        model.decode_loop(first, PROMPT_LEN, 8)
        _, _ = model.decode_loop(first, PROMPT_LEN, 32)
        st = model.last_stats()
        model.set_profile(False)
        n_lin = 4 * cfgd["n_layers"] + 1
        gemv_ms_tok = st["ms_gemv"] / 32
        achieved = wbytes / (gemv_ms_tok * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "k_linear (fused dequant GEMV, all 4*NL+1 launches of a token)",
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                    "peak_source": peak_src, "algorithmic_bytes_per_launch": wbytes / n_lin,
                    "avg_launch_us": gemv_ms_tok * 1e3 / n_lin,
                    "token_bytes": {"weights": wbytes, "kv_mid_run": kvbytes_mid, "embedding_row": embbytes},
                    "whole_token_frac": token_bytes * value / args.gpus / 1e9 / peak,
                    "per_token_ms": {"gemv": gemv_ms_tok, "attention": st["ms_attn"] / 32, "other": st["ms_other"] / 32}}

    # end to end through the per-token public call, host buffers both ways
    pin_lg, pin_io = hb.PinnedArray(shape["vocab"], np.float32), hb.PinnedArray(2, np.int32)      # page-locked host buffers
    check(L.hx_sync())
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    e2e_steps = 0 if args.no_e2e else max(1, min(args.steps, 2))
    for _ in range(e2e_steps):
        tok = first
        for i in range(NEW_TOKENS):
            tok, lg = model.decode_step(tok, PROMPT_LEN + i, out=pin_lg.array, io=pin_io.array)
    e2e_s = all_max(dist, time.perf_counter() - t0)
    pin_lg.free(); pin_io.free()
    e2e = None if args.no_e2e else {"value": n_seq * e2e_steps * NEW_TOKENS / e2e_s, "unit": "tok/s",
           "h2d_bytes_per_step": NEW_TOKENS * 4, "d2h_bytes_per_step": NEW_TOKENS * (4 + shape["vocab"] * 4),
           "api": "hx_decode_step per token with page-locked host buffers: token id H2D, next id + f32 logits row D2H (what the reference worker reads back)"}

    extras = not args.no_e2e and not args.layers
    # the other half of the path: the NVFP4 quantizer on the single-matrix shape (12288 x 4096 f32), device resident
    quant = None
    if rank == 0 and extras:
        rows, K = 12288, 4096
        kp = L.hx_kpad(K)
        w = (np.random.default_rng(7).standard_normal((rows, K), dtype=np.float32) * np.float32(0.02))
        dw = hb.DeviceBuffer.from_array(w)
        dW, dmic, dts = hb.DeviceBuffer(rows * (kp // 7) * 4), hb.DeviceBuffer(rows * (kp // 16)), hb.DeviceBuffer(4)
        for _ in range(3):
            check(L.hx_quantize_nvfp4(dw.ptr, rows, K, dW.ptr, dmic.ptr, None, dts.ptr, None))
        check(L.hx_sync())
        tq = time.perf_counter()
        nrep = 20
        for _ in range(nrep):
            check(L.hx_quantize_nvfp4(dw.ptr, rows, K, dW.ptr, dmic.ptr, None, dts.ptr, None))
        check(L.hx_sync())
        dtq = (time.perf_counter() - tq) / nrep
        alg = rows * K * 4 + rows * (kp // 7) * 4 + rows * (kp // 16)
        quant = {"shape": [rows, K], "ms": dtq * 1e3, "gelem_per_s": rows * K / dtq / 1e9,
                 "algorithmic_bytes": alg, "achieved_gb_s": alg / dtq / 1e9, "frac_of_hbm_peak": alg / dtq / 1e9 / peak,
                 "note": "amax pass + quantize pass (k_amax, k_quantize), bit-exact with the reference quantizer; algorithmic bytes = "
                         "one f32 read of the tensor + the committed layout written; the second read of the tensor mostly misses L2 (201 MB)"}
        for b in (dw, dW, dmic, dts):
            b.free()

    # what the tensor pipe can issue for the MMA of this library (no vendor figure exists for it at small N): the
    # denominator of the batched GEMM's tensor-side roofline
    tprobe = None
    if rank == 0 and extras:
        c16, _ = hb.probe_mxf4_rate(16, True)
        c256, tf256 = hb.probe_mxf4_rate(256, False)
        c256s, tf256s = hb.probe_mxf4_rate(256, True)
        lin_weights = (algorithmic_bytes_per_token(shape, 0)[0] / 0.5625) - shape["vocab"] * shape["d_model"]      # all linears but the head
        useful = PROMPT_LEN / prefill_s * 2.0 * lin_weights / 1e12
        tprobe = {"mma": "tcgen05.mma kind::mxf4nvf4 block16, M128 x N x K64, operands in shared memory, one issuing thread per SM",
                  "clk_per_mma_n16_with_scale_copies": c16, "clk_per_mma_n256": c256, "clk_per_mma_n256_with_scale_copies": c256s,
                  "attainable_tflops_n256": tf256, "attainable_tflops_n256_with_scale_copies": tf256s,
                  "prefill_useful_tflops": useful, "prefill_issued_tflops": useful * 10.0,
                  "prefill_issued_frac_of_attainable": useful * 10.0 / (tf256s * 240.0 / 256.0),
                  "note": "the prefill issues ten digit columns per activation (balanced base 9), 240 columns per MMA, so its issued work is 10 x the useful work"}

    # GPT-2-124M shape, all linears NVFP4, 32-token prompt + 128 greedy tokens, batch 1
    gpt2 = None
    if rank == 0 and extras and not tp:
        gs = dict(hb.GPT2_124M)
        grng = np.random.default_rng(5)
        gn = lambda *sh: grng.standard_normal(sh, dtype=np.float32) * np.float32(0.02)
        one = lambda k: np.ones(k, np.float32)
        DMg, DFg = gs["d_model"], gs["d_ff"]
        gw = dict(wte=gn(gs["vocab"], DMg), wpe=gn(gs["max_ctx"], DMg), lnf_g=one(DMg), lnf_b=np.zeros(DMg, np.float32),
                  layers=[dict(ln1_g=one(DMg), ln1_b=np.zeros(DMg, np.float32), w_qkv=gn(3 * DMg, DMg), b_qkv=gn(3 * DMg),
                               w_proj=gn(DMg, DMg), b_proj=gn(DMg), ln2_g=one(DMg), ln2_b=np.zeros(DMg, np.float32),
                               w_fc=gn(DFg, DMg), b_fc=gn(DFg), w_proj2=gn(DMg, DFg), b_proj2=gn(DMg)) for _ in range(gs["n_layers"])])
        g2 = hb.Model.gpt2(gs, gw, kv_cap=192)
        gp = grng.integers(0, gs["vocab"], 32).astype(np.int32)
        g2.generate(gp, 16)
        _, gms_p, gms_d = g2.generate(gp, 128)
        gpt2 = {"shape": "gpt2-124m", "prompt": 32, "new_tokens": 128, "decode_tok_per_s": 127 / (gms_d * 1e-3), "prefill_ms": gms_p,
                "engine": g2.engine(), "note": "per-op kernels in one CUDA graph per token (LayerNorm/bias/GELU fused into the NVFP4 GEMV)"}
        g2.close(); del gw

    # prompt-lookup speculative decode: the same tokens as plain greedy are required.  (a) the benchmark's own model:
    # with random weights and a 151 936-token vocabulary nothing ever repeats, so the drafter finds nothing and the
    # path is the plain one; (b) a narrow 3-layer model (the width of the parity tests) whose greedy continuation falls
    # into loops, like a real model quoting its prompt: drafts hit and several tokens come out of one verify forward.
    spec = None
    if rank == 0 and extras and not tp:
        def spec_run(mdl, vocab, n_sp):
            base = np.random.default_rng(11).integers(0, vocab, 24).astype(np.int32)
            sp_prompt = np.concatenate([base, base, base[:16]]).astype(np.int32)
            mdl.reset()
            plain_ids, _, plain_ms = mdl.generate(sp_prompt, n_sp)
            mdl.reset()
            spec_ids, st, _, spec_ms = mdl.generate_spec(sp_prompt, n_sp)
            return {"prompt": int(len(sp_prompt)), "new_tokens": n_sp, "tokens_identical_to_greedy": bool(list(plain_ids) == list(spec_ids)),
                    "plain_tok_per_s": (n_sp - 1) / (plain_ms * 1e-3), "spec_tok_per_s": (n_sp - 1) / (spec_ms * 1e-3), "counters": st,
                    "tokens_per_verify_forward": st["emitted"] / st["forwards"] if st["forwards"] else None}
        spec = {"benchmark_model": spec_run(model, shape["vocab"], 96)}
        small = dict(n_layers=3, d_model=512, n_heads=4, n_kv_heads=1, head_dim=128, d_ff=768, vocab=2011)
        sm = hb.Model.synth(small, seed=3, kv_cap=512)
        spec["small_model_d512_vocab_2011"] = spec_run(sm, small["vocab"], 256)
        sm.close()
        spec["note"] = ("a verify forward is one chunk of the batched prefill path (the last token and the drafts, 16 rows at most) plus the head on every row; it pays when "
                        "about three drafted tokens are accepted per hit")

    cpu = parity = None
    if rank == 0 and args.gpus == 1 and not args.no_cpu_baseline:      # reported at N = 1 only
        cpu, parity = cpu_baseline_with_parity(model)
    model.close()

    ref_gpu = batch64 = tpl = None
    if extras and not tp:
        if rank == 0 and args.gpus == 1 and not args.no_reference_gpu:
            ref_gpu = reference_gpu_leg(hb, args.reference_gpu_layers)
        if dist is not None:
            dist.barrier()
        if not args.no_batch64:
            batch64 = batch64_leg(hb, L, check, dist, rank, args.gpus, shape)
        if not args.no_tp_leg:
            tpl = tp_leg(hb, L, check, dist, rank, args.gpus, peak)
    if rank == 0:
        line = {"metric": "nvfp4_decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_max / args.steps, "higher_is_better": True, "scaling": "strong" if tp else "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": WORKLOAD.replace("qwen3-8b", "qwen3-32b") if args.model == "32b" else WORKLOAD, "weights": "nvfp4 (e2m1 + e4m3/16 + f32 tensor scale), HBM resident",
                           "kv_cache": "f32", "engine": engine, "layers": cfgd["n_layers"],
                           "parallelism": (f"tp{args.gpus} (one sequence, exchange inside the decode kernel over NVLink peer memory)" if tp else
                                           f"replicas x{args.gpus} (one sequence per GPU)") if args.gpus > 1 else "single GPU",
                           "l2": "weights (4.26 GB per token) exceed the 126 MB L2, no flush needed",
                           "tokens_per_step": NEW_TOKENS, "weight_bytes_decode_layout": dbytes, "weight_bytes_committed_layout": cbytes},
                "roofline": roofline, "cpu_baseline": cpu, "parity": parity, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
                "reference_gpu": ref_gpu, "batch64": batch64, "tp": tpl, "speculative": spec, "tensor_probe": tprobe, "quantizer": quant, "gpt2": gpt2,
                "prefill": {"tokens": PROMPT_LEN, "ms": prefill_s * 1e3, "tok_per_s": PROMPT_LEN / prefill_s,
                            "path": "chunks of 64 tokens, one tcgen05 block-scaled GEMM per linear (ten base-9 digit columns per activation), host ids in"},
                "ms_per_token": ms_max / args.steps / NEW_TOKENS, "last_tokens": [int(t) for t in toks[-4:]]}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def chunk_probe(args):
    """A small, bounded case of the chunk kernels (k_gemm_tc at 64 tokens, k_pf_attn in both modes) for profiler captures."""
    import helix_b200 as hb
    shape = dict(hb.QWEN3_8B)
    shape["n_layers"] = args.layers or 2
    ctx = 2048
    m = hb.Model.synth(shape, seed=1, kv_cap=ctx + 256, batch=64)
    m.fill_kv(ctx, 7)
    ids = np.random.default_rng(1).integers(0, shape["vocab"], 64).astype(np.int32)
    nxt = ids
    for _ in range(2):
        nxt = m.decode_batch(ids, np.full(64, ctx, np.int32))
    prompt = np.random.default_rng(2).integers(0, shape["vocab"], 512).astype(np.int32)
    first = m.prefill_seq(0, prompt)
    m.close()
    print(json.dumps({"probe": "chunk path", "layers": shape["n_layers"], "sequences": 64, "context": ctx,
                      "next": [int(v) for v in nxt[:4]], "prefill_next": int(first)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parallelism", default="replicas", choices=["replicas", "tp"],
                    help="N > 1: independent replicas (one sequence per GPU, weak scaling) or one tensor-parallel group (strong)")
    ap.add_argument("--model", default="8b", choices=["8b", "32b"], help="Qwen3-8B shape (the headline workload) or Qwen3-32B shape")
    ap.add_argument("--no-e2e", action="store_true", help="skip the per-token host-buffer loop and the side legs (profiler captures)")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip the run of the reference's own GPU worker")
    ap.add_argument("--reference-gpu-layers", type=int, default=4, help="depth of the model the reference GPU worker is timed on")
    ap.add_argument("--no-batch64", action="store_true", help="skip the 64-sequence batched-throughput leg")
    ap.add_argument("--no-tp-leg", action="store_true", help="skip the Qwen3-32B-shape tensor-parallel leg")
    ap.add_argument("--layers", type=int, default=0, help="reduced depth for profiler captures (0 = the full 36)")
    ap.add_argument("--new-tokens", type=int, default=0, help="tokens per step for profiler captures (0 = 256)")
    ap.add_argument("--prompt-len", type=int, default=0, help="prompt length for profiler captures (0 = 512)")
    ap.add_argument("--chunk-probe", action="store_true",
                    help="profiler capture of the chunk path at --layers depth (default 2): 64 sequences at 2048 positions "
                         "(synthetic KV rows), two batched decode steps, then a 512-token prefill; prints no bench line")
    args = ap.parse_args()
    global PROMPT_LEN, NEW_TOKENS
    if args.new_tokens:
        NEW_TOKENS = args.new_tokens
    if args.prompt_len:
        PROMPT_LEN = args.prompt_len
    reduced = bool(args.layers or args.new_tokens or args.prompt_len)
    args.warmup = max(args.warmup, 3) if (args.impl == "ours" and not reduced) else args.warmup
    if args.chunk_probe:
        chunk_probe(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
