"""ctypes binding of libhelix_b200.so (see include/helix_b200.h for the contract of each call)."""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


def lib_path():
    return os.path.join(_HERE, "libhelix_b200.so")


def fatbin_path():
    return os.path.join(_HERE, "helix_b200_kernels.fatbin")


class HxError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"helix_b200 error {code}: {msg}")
        self.code = code
        self.msg = msg


class HxConfig(C.Structure):
    _fields_ = [("arch", C.c_int32), ("n_layers", C.c_int32), ("d_model", C.c_int32), ("n_heads", C.c_int32),
                ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("d_ff", C.c_int32), ("vocab", C.c_int32),
                ("max_ctx", C.c_int32), ("rope_theta", C.c_float), ("norm_eps", C.c_float), ("qk_norm", C.c_int32)]

    def as_dict(self):
        return {k: getattr(self, k) for k, _ in self._fields_}


class HxStepStats(C.Structure):
    _fields_ = [("ms_total", C.c_float), ("kernel_launches", C.c_uint32), ("ms_gemv", C.c_float),
                ("ms_attn", C.c_float), ("ms_other", C.c_float)]


class HxPackReport(C.Structure):
    _fields_ = [("tensors", C.c_int), ("packed", C.c_int), ("bytes", C.c_uint64), ("worst_rms", C.c_double), ("worst_name", C.c_char * 128),
                ("f32_exact", C.c_int), ("verified", C.c_int), ("ms_pack", C.c_float), ("ms_verify", C.c_float)]


class HxSampleConfig(C.Structure):
    _fields_ = [("temperature", C.c_double), ("top_p", C.c_double), ("min_p", C.c_double), ("rep_penalty", C.c_double),
                ("freq_penalty", C.c_double), ("pres_penalty", C.c_double), ("top_k", C.c_int), ("seed", C.c_uint64)]


class HxSpecConfig(C.Structure):
    _fields_ = [("k_max", C.c_int), ("k_min", C.c_int), ("m", C.c_int), ("min_margin", C.c_float)]


class HxSpecStats(C.Structure):
    _fields_ = [(n, C.c_long) for n in ("steps", "hits", "drafted", "accepted", "emitted", "forwards", "single_steps", "near_ties")]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


def _cfg(n_layers, d_model, n_heads, n_kv_heads, head_dim, d_ff, vocab, max_ctx=40960, theta=1e6, eps=1e-5):
    return HxConfig(1, n_layers, d_model, n_heads, n_kv_heads, head_dim, d_ff, vocab, max_ctx, theta, eps, 1)


# Shapes named by the benchmark configurations.  norm_eps is the value the reference's kernels compute
# with (1e-5, baked into its RMSNorm kernel), not the 1e-6 a Qwen3 config file states.
QWEN3_8B = dict(n_layers=36, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, d_ff=12288, vocab=151936)
QWEN3_32B = dict(n_layers=64, d_model=5120, n_heads=64, n_kv_heads=8, head_dim=128, d_ff=25600, vocab=151936)

GPT2_124M = dict(n_layers=12, d_model=768, n_heads=12, d_ff=3072, vocab=50257, max_ctx=1024)
_GPT2_LAYER_FIELDS = ("ln1_g", "ln1_b", "w_qkv", "b_qkv", "w_proj", "b_proj", "ln2_g", "ln2_b", "w_fc", "b_fc", "w_proj2", "b_proj2")


class HxGpt2Layer(C.Structure):
    _fields_ = [(k, C.c_void_p) for k in _GPT2_LAYER_FIELDS]


class HxGpt2Weights(C.Structure):
    _fields_ = [("wte", C.c_void_p), ("wpe", C.c_void_p), ("lnf_g", C.c_void_p), ("lnf_b", C.c_void_p), ("layers", C.POINTER(HxGpt2Layer))]


HX_LOAD_KEEP_COMMITTED = 1
HX_LOAD_VERIFY_SHA = 2
HX_LOAD_FILE_EPS = 4

_lib = None

_SIGS = {
    "hx_last_error": (C.c_char_p, []),
    "hx_version": (C.c_char_p, []),
    "hx_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "hx_set_device": (C.c_int, [C.c_int]),
    "hx_malloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "hx_free": (C.c_int, [C.c_void_p]),
    "hx_memcpy_h2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "hx_memcpy_d2h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "hx_memset": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t]),
    "hx_sync": (C.c_int, []),
    "hx_host_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "hx_host_free": (C.c_int, [C.c_void_p]),
    "hx_launch_count": (C.c_ulonglong, []),
    "hx_e2m1_decode": (C.c_float, [C.c_int]),
    "hx_e2m1_encode": (C.c_int, [C.c_float]),
    "hx_e4m3_decode": (C.c_float, [C.c_int]),
    "hx_e4m3_encode": (C.c_int, [C.c_float]),
    "hx_kpad": (C.c_int, [C.c_int]),
    "hx_kd": (C.c_int, [C.c_int]),
    "hx_quantize_nvfp4": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "hx_quantize_nvfp4_noalloc": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "hx_noalloc_max_rows": (C.c_int, []),
    "hx_quantize_nvfp4_host": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "hx_dequant_nvfp4": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "hx_pack_micro": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "hx_gemv_nvfp4": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "hx_roundtrip_host": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]),
    "hx_repack_d16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "hx_gemv_d16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "hx_gemm_nvfp4_tc": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "hx_gemm_nvfp4_tc_bench": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "hx_sha256": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "hx_sha256_hex": (C.c_int, [C.c_void_p, C.c_size_t, C.c_char_p]),
    "hx_sha256_file": (C.c_int, [C.c_char_p, C.c_char_p]),
    "hx_receipt_emit": (C.c_int, [C.c_char_p, C.c_char_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_double, C.c_char_p]),
    "hx_receipt_check": (C.c_int, [C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p]),
    "hx_model_load": (C.c_int, [C.POINTER(C.c_void_p), C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "hx_model_synth": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(HxConfig), C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "hx_model_free": (C.c_int, [C.c_void_p]),
    "hx_model_config": (C.c_int, [C.c_void_p, C.POINTER(HxConfig)]),
    "hx_model_weight_bytes": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "hx_model_v3_size": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "hx_model_v3_export": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64]),
    "hx_model_v3_save": (C.c_int, [C.c_void_p, C.c_char_p]),
    "hx_model_sha256": (C.c_int, [C.c_void_p, C.c_char_p]),
    "hx_model_reset": (C.c_int, [C.c_void_p]),
    "hx_decode_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "hx_prefill": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "hx_prefill_seq": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "hx_generate_greedy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "hx_tokenizer_load": (C.c_int, [C.POINTER(C.c_void_p), C.c_char_p, C.c_char_p]),
    "hx_tokenizer_free": (C.c_int, [C.c_void_p]),
    "hx_tokenizer_vocab_size": (C.c_int, [C.c_void_p]),
    "hx_tokenizer_encode": (C.c_int, [C.c_void_p, C.c_char_p, C.c_size_t, C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_int)]),
    "hx_tokenizer_decode": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "hx_serve_text": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "hx_sampler_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int]),
    "hx_sampler_configure": (C.c_int, [C.c_void_p, C.POINTER(HxSampleConfig)]),
    "hx_sampler_reset": (C.c_int, [C.c_void_p, C.POINTER(HxSampleConfig), C.c_void_p, C.c_int]),
    "hx_sampler_next": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]),
    "hx_sampler_count": (C.c_int, [C.c_void_p, C.c_int32]),
    "hx_sampler_free": (C.c_int, [C.c_void_p]),
    "hx_serve": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "hx_probe_mxf4_rate": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "hx_pack_qwen3": (C.c_int, [C.c_char_p, C.c_char_p, C.c_int, C.POINTER(HxPackReport)]),
    "hx_pld_draft": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "hx_generate_spec": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(HxSpecConfig), C.c_void_p, C.POINTER(HxSpecStats),
                                   C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "hx_model_last_stats": (C.c_int, [C.c_void_p, C.POINTER(HxStepStats)]),
    "hx_model_engine": (C.c_char_p, [C.c_void_p]),
    "hx_model_debug_waits": (C.c_int, [C.c_void_p, C.c_uint, C.c_int]),
    "hx_model_gpt2": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(HxConfig), C.POINTER(HxGpt2Weights), C.c_int]),
    "hx_decode_batch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "hx_decode_batch_loop": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_float)]),
    "hx_model_tp_handle": (C.c_int, [C.c_void_p, C.c_void_p]),
    "hx_model_tp_connect": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int]),
    "hx_model_set_profile": (C.c_int, [C.c_void_p, C.c_int]),
    "hx_decode_loop": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_float)]),
    "hx_model_fill_kv": (C.c_int, [C.c_void_p, C.c_int, C.c_uint64]),
    "hx_model_kv_read": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "hx_model_kv_write": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "hx_image_open": (C.c_int, [C.POINTER(C.c_void_p), C.c_char_p]),
    "hx_image_launch": (C.c_int, [C.c_void_p, C.c_char_p, C.c_uint, C.c_uint, C.c_uint, C.c_uint, C.c_uint, C.c_uint, C.c_void_p]),
    "hx_image_close": (C.c_int, [C.c_void_p]),
}


def lib():
    """Load the shared library; raises HxError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    p = lib_path()
    if not os.path.exists(p):
        raise HxError(-1, f"{p} is missing: build it with `make -C helix_b200/csrc` (no CPU fallback exists)")
    L = C.CDLL(p)
    for name, (res, args) in _SIGS.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def check(rc):
    if rc != 0:
        raise HxError(rc, lib().hx_last_error().decode(errors="replace"))


def launch_count():
    return int(lib().hx_launch_count())


class PinnedArray:
    """Page-locked host memory (hx_host_alloc) seen as a numpy array: the host side of the per-token calls."""

    def __init__(self, count, dtype=np.float32):
        dt = np.dtype(dtype)
        self.ptr = C.c_void_p()
        self.nbytes = int(count) * dt.itemsize
        check(lib().hx_host_alloc(C.byref(self.ptr), self.nbytes))
        self.array = np.ctypeslib.as_array(C.cast(self.ptr, C.POINTER(C.c_uint8)), shape=(self.nbytes,)).view(dt)

    def free(self):
        if self.ptr:
            self.array = None
            check(lib().hx_host_free(self.ptr))
            self.ptr = C.c_void_p()


class DeviceBuffer:
    """A device allocation owned through the C ABI."""

    def __init__(self, nbytes):
        self.ptr = C.c_void_p()
        self.nbytes = int(nbytes)
        check(lib().hx_malloc(C.byref(self.ptr), self.nbytes))

    @classmethod
    def from_array(cls, a):
        a = np.ascontiguousarray(a)
        b = cls(a.nbytes)
        check(lib().hx_memcpy_h2d(b.ptr, a.ctypes.data, a.nbytes))
        return b

    def zero(self):
        check(lib().hx_memset(self.ptr, 0, self.nbytes))
        return self

    def upload(self, a, offset=0):
        a = np.ascontiguousarray(a)
        check(lib().hx_memcpy_h2d(C.c_void_p(self.ptr.value + offset), a.ctypes.data, a.nbytes))

    def to_array(self, dtype, count=None):
        dt = np.dtype(dtype)
        n = self.nbytes // dt.itemsize if count is None else count
        out = np.empty(n, dt)
        check(lib().hx_memcpy_d2h(out.ctypes.data, self.ptr, n * dt.itemsize))
        return out

    def free(self):
        if self.ptr:
            lib().hx_free(self.ptr)
            self.ptr = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def quantize_host(w):
    """hx_quantize_nvfp4_host: returns (words[rows,Kpad/7] i32, micro[rows,Kpad/16] u8, sc f32, ts)."""
    w = np.ascontiguousarray(w, np.float32)
    rows, K = w.shape
    kp = lib().hx_kpad(K)
    W = np.empty((rows, kp // 7), np.int32)
    mic = np.empty((rows, kp // 16), np.uint8)
    sc = np.empty((rows, kp // 16), np.float32)
    ts = np.empty(1, np.float32)
    check(lib().hx_quantize_nvfp4_host(w.ctypes.data, rows, K, W.ctypes.data, mic.ctypes.data, sc.ctypes.data, ts.ctypes.data))
    return W, mic, sc, float(ts[0])


def roundtrip_host(w, x):
    w = np.ascontiguousarray(w, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    rows, K = w.shape
    y = np.empty(rows, np.float32)
    kp = C.c_int()
    check(lib().hx_roundtrip_host(w.ctypes.data, rows, K, x.ctypes.data, y.ctypes.data, C.byref(kp)))
    return y


class KernelImage:
    """The kernel-entry image loaded and launched the way the reference's C launchers do it."""

    def __init__(self, path=None):
        self.mod = C.c_void_p()
        check(lib().hx_image_open(C.byref(self.mod), (path or fatbin_path()).encode()))

    def launch(self, entry, grid, block, args):
        """args: DeviceBuffer -> its pointer, int -> 32-bit scalar (the reference's kernel ABI has only those)."""
        grid = tuple(grid) + (1,) * (3 - len(grid))
        block = tuple(block) + (1,) * (3 - len(block))
        holders = []
        for a in args:
            holders.append(C.c_void_p(a.ptr.value) if isinstance(a, DeviceBuffer) else C.c_int32(int(a)))
        arr = (C.c_void_p * len(holders))(*[C.cast(C.pointer(h), C.c_void_p) for h in holders])
        check(lib().hx_image_launch(self.mod, entry.encode(), *grid, *block, arr))

    def close(self):
        if self.mod:
            lib().hx_image_close(self.mod)
            self.mod = C.c_void_p()


class Model:
    """hx_model: HBM-resident NVFP4 weights + KV cache + the captured decode step."""

    def __init__(self, handle):
        self.h = handle
        c = HxConfig()
        check(lib().hx_model_config(self.h, C.byref(c)))
        self.cfg = c
        self.vocab = c.vocab

    @classmethod
    def load(cls, path, kv_cap=1024, flags=0, tp_rank=0, tp_size=1, batch=1):
        h = C.c_void_p()
        check(lib().hx_model_load(C.byref(h), path.encode(), kv_cap, batch, flags, tp_rank, tp_size))
        return cls(h)

    @classmethod
    def synth(cls, shape, seed=0, kv_cap=1024, flags=0, eps=1e-5, tp_rank=0, tp_size=1, batch=1):
        cfg = _cfg(eps=eps, **shape)
        h = C.c_void_p()
        check(lib().hx_model_synth(C.byref(h), C.byref(cfg), seed, kv_cap, batch, flags, tp_rank, tp_size))
        return cls(h)

    def decode_batch(self, ids, pos):
        """One token of each sequence i (KV slot i): ids[i] at pos[i]; returns the arg-max tokens."""
        ids = np.ascontiguousarray(ids, np.int32); pos = np.ascontiguousarray(pos, np.int32)
        out = np.zeros(len(ids), np.int32)
        check(lib().hx_decode_batch(self.h, ids.ctypes.data, pos.ctypes.data, len(ids), out.ctypes.data))
        return out

    def decode_batch_loop(self, ids, pos0, n_steps):
        ids = np.ascontiguousarray(ids, np.int32)
        out = np.zeros((n_steps, len(ids)), np.int32)
        ms = C.c_float()
        check(lib().hx_decode_batch_loop(self.h, ids.ctypes.data, pos0, len(ids), n_steps, out.ctypes.data, C.byref(ms)))
        return out, ms.value

    @classmethod
    def gpt2(cls, shape, weights, kv_cap=256):
        """shape: n_layers, d_model, n_heads, d_ff, vocab, max_ctx.  weights: dict with wte, wpe, lnf_g, lnf_b and
        layers = list of dicts with the twelve per-layer tensors, all float32, linears as [out][in]."""
        cfg = HxConfig(0, shape["n_layers"], shape["d_model"], shape["n_heads"], shape["n_heads"],
                       shape["d_model"] // shape["n_heads"], shape["d_ff"], shape["vocab"], shape["max_ctx"], 0.0, 1e-5, 0)
        keep = []

        def ptr(a):
            a = np.ascontiguousarray(a, np.float32); keep.append(a)
            return a.ctypes.data

        lay = (HxGpt2Layer * shape["n_layers"])()
        for i, lw in enumerate(weights["layers"]):
            for k in _GPT2_LAYER_FIELDS:
                setattr(lay[i], k, ptr(lw[k]))
        hw = HxGpt2Weights(ptr(weights["wte"]), ptr(weights["wpe"]), ptr(weights["lnf_g"]), ptr(weights["lnf_b"]), lay)
        h = C.c_void_p()
        check(lib().hx_model_gpt2(C.byref(h), C.byref(cfg), C.byref(hw), kv_cap))
        return cls(h)

    def tp_handle(self):
        """64-byte handle of this shard's exchange buffer (to be gathered from all ranks)."""
        b = (C.c_uint8 * 64)()
        check(lib().hx_model_tp_handle(self.h, b))
        return bytes(b)

    def tp_connect(self, handles):
        """handles: the 64-byte handles of all ranks in rank order."""
        blob = b"".join(handles)
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        check(lib().hx_model_tp_connect(self.h, buf, len(handles)))

    def close(self):
        if self.h:
            lib().hx_model_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def weight_bytes(self):
        a, b = C.c_uint64(), C.c_uint64()
        check(lib().hx_model_weight_bytes(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def decode_step(self, tok, pos, want_logits=False, out=None, io=None):
        """One token.  `out` (float32 array of the vocabulary size, e.g. PinnedArray.array) receives the logits instead of a
        fresh array; `io` (int32 array of two words, pinned) carries the token id in and the next id out."""
        if io is None:
            io = np.zeros(2, np.int32)
        io[0] = tok
        lg = out if out is not None else (np.empty(self.vocab, np.float32) if want_logits else None)
        check(lib().hx_decode_step(self.h, io.ctypes.data, pos, io.ctypes.data + 4, lg.ctypes.data if lg is not None else None))
        return (int(io[1]), lg) if lg is not None else int(io[1])

    def prefill(self, ids, want_logits=False):
        ids = np.ascontiguousarray(ids, np.int32)
        nxt = np.zeros(1, np.int32)
        lg = np.empty(self.vocab, np.float32) if want_logits else None
        check(lib().hx_prefill(self.h, ids.ctypes.data, len(ids), nxt.ctypes.data, lg.ctypes.data if want_logits else None))
        return (int(nxt[0]), lg) if want_logits else int(nxt[0])

    def prefill_seq(self, seq, ids, want_logits=False):
        """Prompt of sequence `seq` of a batch into its KV slot; returns the arg-max token (and the logits)."""
        ids = np.ascontiguousarray(ids, np.int32)
        nxt = np.zeros(1, np.int32)
        lg = np.empty(self.vocab, np.float32) if want_logits else None
        check(lib().hx_prefill_seq(self.h, seq, ids.ctypes.data, len(ids), nxt.ctypes.data, lg.ctypes.data if want_logits else None))
        return (int(nxt[0]), lg) if want_logits else int(nxt[0])

    def reset(self):
        """Forget the cached positions (the next prefill starts a new sequence)."""
        check(lib().hx_model_reset(self.h))

    def generate(self, prompt, n_new):
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.zeros(n_new, np.int32)
        a, b = C.c_float(), C.c_float()
        check(lib().hx_generate_greedy(self.h, prompt.ctypes.data, len(prompt), n_new, out.ctypes.data, C.byref(a), C.byref(b)))
        return out, a.value, b.value

    def generate_spec(self, prompt, n_new, k_max=3, k_min=1, m=6, min_margin=1e-3):
        """Prompt-lookup speculative greedy decode: (tokens, counters, ms_prefill, ms_decode)."""
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.zeros(n_new, np.int32)
        cfg = HxSpecConfig(k_max, k_min, m, min_margin)
        st = HxSpecStats()
        a, b = C.c_float(), C.c_float()
        check(lib().hx_generate_spec(self.h, prompt.ctypes.data, len(prompt), n_new, C.byref(cfg), out.ctypes.data, C.byref(st),
                                     C.byref(a), C.byref(b)))
        return out, st.as_dict(), a.value, b.value

    def decode_loop(self, tok, pos0, n_steps):
        ids = np.array([tok], np.int32)
        out = np.zeros(n_steps, np.int32)
        ms = C.c_float()
        check(lib().hx_decode_loop(self.h, ids.ctypes.data, pos0, n_steps, out.ctypes.data, C.byref(ms)))
        return out, ms.value

    def engine(self):
        return lib().hx_model_engine(self.h).decode()

    def debug_waits(self, wait_limit=0, inject_stall=False):
        check(lib().hx_model_debug_waits(self.h, int(wait_limit), 1 if inject_stall else 0))

    def set_profile(self, on):
        check(lib().hx_model_set_profile(self.h, 1 if on else 0))

    def last_stats(self):
        st = HxStepStats()
        check(lib().hx_model_last_stats(self.h, C.byref(st)))
        return {k: getattr(st, k) for k, _ in st._fields_}

    def fill_kv(self, T, seed=0):
        check(lib().hx_model_fill_kv(self.h, T, seed))

    def kv_read(self, layer, kv_head, pos0, n, seq=0):
        """Cached K and V rows [pos0, pos0 + n) of one (layer, kv head): two [n, head_dim] float32 arrays."""
        k = np.empty((n, self.cfg.head_dim), np.float32); v = np.empty_like(k)
        check(lib().hx_model_kv_read(self.h, seq, layer, kv_head, pos0, n, k.ctypes.data, v.ctypes.data))
        return k, v

    def kv_write(self, layer, kv_head, pos0, k, v, seq=0):
        k = np.ascontiguousarray(k, np.float32); v = np.ascontiguousarray(v, np.float32)
        check(lib().hx_model_kv_write(self.h, seq, layer, kv_head, pos0, k.shape[0], k.ctypes.data, v.ctypes.data))

    def v3_image(self):
        n = C.c_uint64()
        check(lib().hx_model_v3_size(self.h, C.byref(n)))
        buf = np.empty(n.value, np.uint8)
        check(lib().hx_model_v3_export(self.h, buf.ctypes.data, n.value))
        return buf

    def save_v3(self, path):
        check(lib().hx_model_v3_save(self.h, path.encode()))

    def sha256(self):
        b = C.create_string_buffer(65)
        check(lib().hx_model_sha256(self.h, b))
        return b.value.decode()


def pld_draft(ids, k_min=1, k_max=3, m=6):
    """The host-side n-gram drafter of the speculative decoder: the draft tokens for the sequence `ids`."""
    ids = np.ascontiguousarray(ids, np.int32)
    out = np.zeros(16, np.int32)
    n = lib().hx_pld_draft(ids.ctypes.data, len(ids), k_min, k_max, m, out.ctypes.data)
    return out[:n].copy()


def pack_qwen3(model_dir, out_path, verify=True):
    """Safetensors checkpoint directory -> HXGW v3 NVFP4 file on the GPU; returns the report as a dict."""
    rep = HxPackReport()
    check(lib().hx_pack_qwen3(os.fsencode(model_dir), os.fsencode(out_path), 1 if verify else 0, C.byref(rep)))
    return dict(tensors=rep.tensors, packed=rep.packed, bytes=rep.bytes, worst_rms=rep.worst_rms, worst_name=rep.worst_name.decode(),
                f32_exact=bool(rep.f32_exact), verified=bool(rep.verified), ms_pack=rep.ms_pack, ms_verify=rep.ms_verify)


def probe_mxf4_rate(ncols, with_scale_copies=False):
    """(SM cycles per M128 x N x K64 block-scaled FP4 MMA, TFLOP/s over all SMs) measured on the current device."""
    clk, tf = C.c_double(), C.c_double()
    check(lib().hx_probe_mxf4_rate(int(ncols), 1 if with_scale_copies else 0, C.byref(clk), C.byref(tf)))
    return clk.value, tf.value


def worker_path():
    """The serve worker process (hx_worker <weights> --serve [--emit-fd N] [--max-ctx M])."""
    return os.path.join(_HERE, "hx_worker")


class Sampler:
    """The reference's seeded sampler on host logits (include/helix_b200.h, hx_sampler_*)."""

    def __init__(self, vocab):
        self.h = C.c_void_p()
        check(lib().hx_sampler_create(C.byref(self.h), vocab))

    def reset(self, prompt=(), temperature=0.0, top_p=1.0, min_p=0.0, rep_penalty=1.0, freq_penalty=0.0, pres_penalty=0.0, top_k=0, seed=0):
        cfg = HxSampleConfig(temperature, top_p, min_p, rep_penalty, freq_penalty, pres_penalty, top_k, seed)
        ids = np.ascontiguousarray(prompt, np.int32)
        check(lib().hx_sampler_reset(self.h, C.byref(cfg), ids.ctypes.data, len(ids)))

    def configure(self, temperature=0.0, top_p=1.0, min_p=0.0, rep_penalty=1.0, freq_penalty=0.0, pres_penalty=0.0, top_k=0, seed=0):
        cfg = HxSampleConfig(temperature, top_p, min_p, rep_penalty, freq_penalty, pres_penalty, top_k, seed)
        check(lib().hx_sampler_configure(self.h, C.byref(cfg)))

    def next(self, logits):
        lg = np.ascontiguousarray(logits, np.float32)
        out = C.c_int32()
        check(lib().hx_sampler_next(self.h, lg.ctypes.data, C.byref(out)))
        return int(out.value)

    def count(self, tok):
        check(lib().hx_sampler_count(self.h, int(tok)))

    def close(self):
        if self.h:
            lib().hx_sampler_free(self.h)
            self.h = None


class Tokenizer:
    """GPT-2 byte-level BPE over a vocab.json and a merges.txt (include/helix_b200.h, hx_tokenizer_*)."""

    def __init__(self, vocab_json, merges_txt):
        self.h = C.c_void_p()
        check(lib().hx_tokenizer_load(C.byref(self.h), os.fsencode(vocab_json), os.fsencode(merges_txt)))

    def vocab_size(self):
        return lib().hx_tokenizer_vocab_size(self.h)

    def encode(self, text, with_specials=False):
        data = text if isinstance(text, (bytes, bytearray)) else text.encode("utf-8")
        ids = np.zeros(len(data) + 8, np.int32)
        n = C.c_int()
        check(lib().hx_tokenizer_encode(self.h, bytes(data), len(data), 1 if with_specials else 0, ids.ctypes.data, len(ids), C.byref(n)))
        return ids[:n.value].copy()

    def decode(self, ids):
        ids = np.ascontiguousarray(ids, np.int32)
        n = C.c_size_t()
        lib().hx_tokenizer_decode(self.h, ids.ctypes.data, len(ids), None, 0, C.byref(n))      # sizes the text
        buf = C.create_string_buffer(max(1, n.value))
        if n.value:
            check(lib().hx_tokenizer_decode(self.h, ids.ctypes.data, len(ids), buf, n.value, C.byref(n)))
        return buf.raw[:n.value]

    def close(self):
        if self.h:
            lib().hx_tokenizer_free(self.h)
            self.h = None
