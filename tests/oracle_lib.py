"""ctypes access to the CPU checker (oracle/hx_oracle.c) and, when it has been built, to the
reference's own quantizer compiled unmodified (oracle/ref_wrap.c -> oracle/_ref/libhelix_ref.so).

Test infrastructure only: nothing in the shipped package imports this module.
"""
import ctypes as C
import os
import struct
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "_build", "libhx_oracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libhelix_ref.so")
REF_PACK = os.path.join(ORACLE_DIR, "_ref", "gpt2_pack")
REF_INFER = os.path.join(ORACLE_DIR, "_ref", "gpt2_infer")
REF_TOK = os.path.join(ORACLE_DIR, "_ref", "gpt2_tok")
REF_INFER_SERVE = os.path.join(ORACLE_DIR, "_ref", "gpt2_infer_serve")

f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")


def build_oracle():
    src = os.path.join(ORACLE_DIR, "hx_oracle.c")
    if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", ORACLE_DIR, "all"])
    return ORACLE_SO


_orc = None


def oracle():
    global _orc
    if _orc is not None:
        return _orc
    lib = C.CDLL(build_oracle())
    lib.orc_e2m1_decode.restype = C.c_float
    lib.orc_e2m1_decode.argtypes = [C.c_int]
    lib.orc_e2m1_encode.argtypes = [C.c_float]
    lib.orc_e2m1_encode_ref.argtypes = [C.c_float]
    lib.orc_e4m3_decode.restype = C.c_float
    lib.orc_e4m3_decode.argtypes = [C.c_int]
    lib.orc_e4m3_encode.argtypes = [C.c_float]
    lib.orc_kpad.argtypes = [C.c_int]
    lib.orc_nvfp4_quantize.argtypes = [f32p, C.c_int, C.c_int, i32p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.orc_nvfp4_dequant_micro.argtypes = [i32p, u8p, C.c_float, f32p, C.c_int, C.c_int]
    lib.orc_nvfp4_dequant_sc.argtypes = [i32p, f32p, f32p, C.c_int, C.c_int]
    lib.orc_pack_micro.argtypes = [u8p, C.c_long, C.c_int, i32p]
    lib.orc_sha256_hex.argtypes = [C.c_void_p, C.c_size_t, C.c_char_p]
    lib.orc_rmsnorm.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_float]
    lib.orc_layernorm.argtypes = [f32p, f32p, f32p, f32p, C.c_int, C.c_int, C.c_float]
    lib.orc_rope_tables.argtypes = [f32p, f32p, C.c_int, C.c_int, C.c_double]
    lib.orc_rope_rot.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int]
    lib.orc_silu_mul.argtypes = [f32p, f32p, f32p, C.c_int]
    lib.orc_gelu.argtypes = [f32p, f32p, C.c_int]
    lib.orc_softmax_row.argtypes = [f32p, f32p, C.c_int, C.c_int]
    lib.orc_softmax_causal_offset.argtypes = [f32p, f32p, C.c_int, C.c_int, C.c_int]
    lib.orc_gemv_abt.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int]
    lib.orc_gemv_ab.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int]
    lib.orc_argmax.argtypes = [f32p, C.c_int]
    lib.orc_gemv_packed.argtypes = [f32p, i32p, u8p, C.c_float, f32p, C.c_int, C.c_int]
    lib.orc_gemv_packed_warp_order.argtypes = [f32p, i32p, u8p, C.c_float, f32p, C.c_int, C.c_int]
    lib.orc_decode_attn_online.argtypes = [f32p, f32p, f32p, f32p, C.c_float, C.c_int, C.c_int, C.c_int,
                                           C.c_long, C.c_int, C.c_long]
    lib.orc_v3_validate.argtypes = [C.c_void_p, C.c_size_t]
    lib.orc_model_open.restype = C.c_void_p
    lib.orc_model_open.argtypes = [C.c_char_p, C.c_int, C.c_int]
    lib.orc_model_open_image.restype = C.c_void_p
    lib.orc_model_open_image.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_int]
    lib.orc_num_threads.restype = C.c_int
    lib.orc_model_close.argtypes = [C.c_void_p]
    lib.orc_model_reset.argtypes = [C.c_void_p]
    lib.orc_model_kv_set.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, f32p, f32p]
    lib.orc_model_dims.argtypes = [C.c_void_p, i32p]
    lib.orc_model_decode.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    lib.orc_model_prefill.argtypes = [C.c_void_p, i32p, C.c_int, C.c_void_p]
    lib.orc_model_generate.argtypes = [C.c_void_p, i32p, C.c_int, C.c_int, i32p, C.c_void_p]
    lib.orc_pld_draft.argtypes = [i32p, C.c_int, C.c_int, C.c_int, C.c_int, i32p]
    lib.orc_pcg_seed.argtypes = [C.c_uint64]; lib.orc_pcg_seed.restype = None
    lib.orc_pcg_next.argtypes = []; lib.orc_pcg_next.restype = C.c_uint32
    lib.orc_sample_next.argtypes = [f32p, C.c_int, C.c_void_p] + [C.c_double] * 6 + [C.c_int]
    lib.orc_sample_next.restype = C.c_int
    lib.orc_pld_draft.restype = C.c_int
    lib.orc_spec_counters.argtypes = [i32p, C.c_int, i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.orc_spec_counters.restype = None
    _orc = lib
    return lib


_ref = None


def reference():
    """The reference quantizer compiled from its own sources, or None when it was not built."""
    global _ref
    if _ref is not None:
        return _ref
    if not os.path.exists(REF_SO):
        return None
    lib = C.CDLL(REF_SO)
    lib.ref_e2m1_decode.restype = C.c_float
    lib.ref_e2m1_decode.argtypes = [C.c_int]
    lib.ref_e2m1_encode.argtypes = [C.c_float]
    lib.ref_e2m1_encode_ref.argtypes = [C.c_float]
    lib.ref_e4m3_decode.restype = C.c_float
    lib.ref_e4m3_decode.argtypes = [C.c_int]
    lib.ref_e4m3_encode.argtypes = [C.c_float]
    lib.ref_nvfp4_quantize.argtypes = [f32p, C.c_int, C.c_int, i32p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ref_nvfp4_host_dequant.argtypes = [i32p, f32p, f32p, C.c_int, C.c_int]
    _ref = lib
    return lib


def kpad(K):
    return ((K + 111) // 112) * 112


def quantize(w, lib=None, fn="orc_nvfp4_quantize"):
    """Quantize a [rows, K] f32 matrix; returns (words[rows,Kpad/7] i32, micro[rows,Kpad/16] u8, ts, sc f32)."""
    lib = lib or oracle()
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, K = w.shape
    kp = kpad(K)
    W = np.zeros((rows, kp // 7), np.int32)
    mic = np.zeros((rows, kp // 16), np.uint8)
    sc = np.zeros((rows, kp // 16), np.float32)
    ts = np.zeros(1, np.float32)
    got = getattr(lib, fn)(w, rows, K, W, sc.ctypes.data, mic.ctypes.data, ts.ctypes.data)
    assert got == kp
    return W, mic, float(ts[0]), sc


def dequant_micro(W, mic, ts):
    rows, kwords = W.shape
    out = np.zeros((rows, kwords * 7), np.float32)
    oracle().orc_nvfp4_dequant_micro(W, mic, np.float32(ts), out, rows, kwords * 7)
    return out


def sha256_hex(data: bytes) -> str:
    buf = C.create_string_buffer(65)
    oracle().orc_sha256_hex(data, len(data), buf)
    return buf.value.decode()


# ---------------------------------------------------------------------------------------------
# HXGW v3 writer (numpy restatement of pack_qwen3's layout, helixc/runtime/gpt2_pack.c:622-680):
# 64-byte header, n_tensors 32-byte descriptors, data in build order.
# ---------------------------------------------------------------------------------------------
def qwen3_tensor_order(cfg):
    """(name, shape, packed) in the order of build_order_llama(qwen3=1), gpt2_pack.c:255-281."""
    NL, DM, NH, NKV, DH, DFF, NV = (cfg[k] for k in ("NL", "DM", "NH", "NKV", "DH", "DFF", "NV"))
    QD, KVD = NH * DH, NKV * DH
    order = []
    for L in range(NL):
        p = f"model.layers.{L}."
        order += [
            (p + "input_layernorm.weight", (DM,), False),
            (p + "self_attn.q_proj.weight", (QD, DM), True),
            (p + "self_attn.q_norm.weight", (DH,), False),
            (p + "self_attn.k_proj.weight", (KVD, DM), True),
            (p + "self_attn.k_norm.weight", (DH,), False),
            (p + "self_attn.v_proj.weight", (KVD, DM), True),
            (p + "self_attn.o_proj.weight", (DM, QD), True),
            (p + "post_attention_layernorm.weight", (DM,), False),
            (p + "mlp.gate_proj.weight", (DFF, DM), True),
            (p + "mlp.up_proj.weight", (DFF, DM), True),
            (p + "mlp.down_proj.weight", (DM, DFF), True),
        ]
    order += [("model.embed_tokens.weight", (NV, DM), False), ("model.norm.weight", (DM,), False),
              ("lm_head.weight", (NV, DM), True)]
    return order


def synth_tensors(cfg, seed=0, norm_jitter=0.1):
    """Seeded synthetic weights: linears and embedding N(0, 0.02); norm gains 1 + jitter*N(0,1) so a
    kernel that drops a gain fails the comparison."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape, packed in qwen3_tensor_order(cfg):
        if len(shape) == 1:
            out[name] = (1.0 + norm_jitter * rng.standard_normal(shape)).astype(np.float32)
        else:
            out[name] = (0.02 * rng.standard_normal(shape)).astype(np.float32)
    return out


def write_v3(path, cfg, tensors, quant=None):
    """Write an HXGW v3 file with the oracle quantizer (or `quant`, same signature as quantize())."""
    quant = quant or quantize
    order = qwen3_tensor_order(cfg)
    nt = len(order)
    descs, blobs = [], []
    cur = 64 + 32 * nt
    for name, shape, packed in order:
        t = np.ascontiguousarray(tensors[name], dtype=np.float32)
        if packed:
            rows, K = shape
            W, mic, ts, _ = quant(t.reshape(rows, K))
            kp = kpad(K)
            wb = rows * (kp // 7) * 4
            descs.append(struct.pack("<IIIIQQ", 1, rows, K, kp, cur, cur + wb))
            blob = W.tobytes() + mic.tobytes() + struct.pack("<f", ts)
        else:
            n = int(np.prod(shape))
            descs.append(struct.pack("<IIIIQQ", 0, 1, n, n, cur, 0))
            blob = t.tobytes()
        blobs.append(blob)
        cur += len(blob)
    hdr = bytearray(64)
    struct.pack_into("<8I", hdr, 0, 0x48584757, 3, cfg["NL"], cfg["DM"], cfg["NH"], cfg["NV"], cfg.get("NC", 40960), cfg["DFF"])
    struct.pack_into("<II", hdr, 40, 1, cfg["NKV"])
    struct.pack_into("<ff", hdr, 48, cfg.get("theta", 1e6), cfg.get("eps", 1e-6))
    struct.pack_into("<II", hdr, 56, cfg["DH"], nt)
    with open(path, "wb") as f:
        f.write(bytes(hdr))
        for d in descs:
            f.write(d)
        for b in blobs:
            f.write(b)
    return cur


def to_bf16_bits(t):
    """f32 -> the upper 16 bits, round to nearest even (what a BF16 checkpoint stores)."""
    u = np.ascontiguousarray(t, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def write_safetensors(path, tensors, dtype="F32"):
    """Minimal safetensors writer (F32 or BF16), enough for the reference importer (gpt2_pack.c:45-207 reads the
    JSON header, dtype, shape and data_offsets)."""
    import json
    hdr, off, blobs = {"__metadata__": {"format": "pt"}}, 0, []
    for name, t in tensors.items():
        b = (to_bf16_bits(t) if dtype == "BF16" else np.ascontiguousarray(t, np.float32)).tobytes()
        hdr[name] = {"dtype": dtype, "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        off += len(b); blobs.append(b)
    js = json.dumps(hdr, separators=(",", ":")).encode()
    js += b" " * ((8 - len(js) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for b in blobs:
            f.write(b)


def write_sharded_checkpoint(d, cfg, tensors, n_shards=2, dtype="BF16"):
    """A checkpoint directory the way the hub lays it out: config.json, model-0000i-of-0000n.safetensors and
    model.safetensors.index.json with the weight_map."""
    import json
    names = list(tensors)
    per = (len(names) + n_shards - 1) // n_shards
    wmap = {}
    for s in range(n_shards):
        fn = "model-%05d-of-%05d.safetensors" % (s + 1, n_shards)
        part = {n: tensors[n] for n in names[s * per:(s + 1) * per]}
        write_safetensors(os.path.join(d, fn), part, dtype)
        for n in part:
            wmap[n] = fn
    json.dump({"metadata": {"total_size": 0}, "weight_map": wmap}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    write_qwen3_config(os.path.join(d, "config.json"), cfg)


def write_qwen3_config(path, cfg):
    import json
    with open(path, "w") as f:
        json.dump({"num_hidden_layers": cfg["NL"], "hidden_size": cfg["DM"], "num_attention_heads": cfg["NH"],
                   "num_key_value_heads": cfg["NKV"], "intermediate_size": cfg["DFF"], "vocab_size": cfg["NV"],
                   "head_dim": cfg["DH"], "max_position_embeddings": cfg.get("NC", 40960),
                   "rope_theta": cfg.get("theta", 1e6), "rms_norm_eps": cfg.get("eps", 1e-6)}, f)


class OracleModel:
    """The fp32 CPU restatement of the worker's decode/prefill over an HXGW v3 file."""

    def __init__(self, path=None, kv_cap=256, use_file_eps=False, image=None):
        self.lib = oracle()
        if image is not None:
            self._image = np.ascontiguousarray(image, np.uint8)      # kept alive: the oracle reads it in place
            self.h = self.lib.orc_model_open_image(self._image.ctypes.data, self._image.nbytes, kv_cap,
                                                   1 if use_file_eps else 0)
        else:
            self.h = self.lib.orc_model_open(path.encode(), kv_cap, 1 if use_file_eps else 0)
        if not self.h:
            raise RuntimeError(f"oracle could not open {path or 'the image'}")
        d = np.zeros(9, np.int32)
        self.lib.orc_model_dims(self.h, d)
        self.NL, self.DM, self.NH, self.NKV, self.DH, self.DFF, self.NV, self.QD, self.KVD = (int(v) for v in d)

    def close(self):
        if self.h:
            self.lib.orc_model_close(self.h)
            self.h = None

    def reset(self):
        self.lib.orc_model_reset(self.h)

    def kv_set(self, layer, kv_head, pos0, k, v):
        k = np.ascontiguousarray(k, np.float32); v = np.ascontiguousarray(v, np.float32)
        assert self.lib.orc_model_kv_set(self.h, layer, kv_head, pos0, k.size // self.DH, k, v) == 0

    def decode(self, tok, pos, want_hidden=False):
        lg = np.zeros(self.NV, np.float32)
        hid = np.zeros(self.DM, np.float32)
        rc = self.lib.orc_model_decode(self.h, int(tok), int(pos), lg.ctypes.data, hid.ctypes.data)
        assert rc == 0
        return (lg, hid) if want_hidden else lg

    def prefill(self, ids):
        ids = np.ascontiguousarray(ids, np.int32)
        lg = np.zeros(self.NV, np.float32)
        assert self.lib.orc_model_prefill(self.h, ids, len(ids), lg.ctypes.data) == 0
        return lg

    def generate(self, ids, n_new):
        ids = np.ascontiguousarray(ids, np.int32)
        out = np.zeros(n_new, np.int32)
        assert self.lib.orc_model_generate(self.h, ids, len(ids), n_new, out, None) == 0
        return out


def pld_draft(ids, k_min=1, k_max=3, m=6):
    ids = np.ascontiguousarray(ids, np.int32)
    out = np.zeros(16, np.int32)
    n = oracle().orc_pld_draft(ids, len(ids), k_min, k_max, m, out)
    return out[:n].copy()


SPEC_COUNTERS = ("steps", "hits", "drafted", "accepted", "emitted", "forwards")


def spec_counters(prompt, greedy, k_min=1, k_max=3, m=6, kv_cap=1 << 30):
    """The reference's [specprof] counters for a prompt whose plain greedy continuation is `greedy`."""
    prompt = np.ascontiguousarray(prompt, np.int32); greedy = np.ascontiguousarray(greedy, np.int32)
    st = (C.c_long * 6)()
    oracle().orc_spec_counters(prompt, len(prompt), greedy, len(greedy), k_min, k_max, m, kv_cap, st)
    return dict(zip(SPEC_COUNTERS, [int(v) for v in st]))
