"""GPT-2 decode (the GPT-2-124M configuration: LayerNorm, learned positions, biases, gelu_new, tied head, all linears NVFP4) on
the GPU against the fp32 CPU restatement of the reference's GPT-2 block fed with the same quantized weights.
The reference has no NVFP4 GPT-2 path: parity is defined as quantizing each linear as [out][in] with the reference
quantizer, dequantizing on the host and running the fp32 GPT-2 arithmetic."""
import ctypes as C

import numpy as np
import pytest

import helix_b200 as hb
import oracle_lib as ol

pytestmark = pytest.mark.gpu
LAYER_KEYS = ("ln1_g", "ln1_b", "w_qkv", "b_qkv", "w_proj", "b_proj", "ln2_g", "ln2_b", "w_fc", "b_fc", "w_proj2", "b_proj2")


def synth(shape, seed):
    rng = np.random.default_rng(seed)
    DM, DFF, NV, CTX = shape["d_model"], shape["d_ff"], shape["vocab"], shape["max_ctx"]
    n = lambda *s: (0.02 * rng.standard_normal(s)).astype(np.float32)
    g = lambda k: (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    layers = [dict(ln1_g=g(DM), ln1_b=n(DM), w_qkv=n(3 * DM, DM), b_qkv=n(3 * DM), w_proj=n(DM, DM), b_proj=n(DM),
                   ln2_g=g(DM), ln2_b=n(DM), w_fc=n(DFF, DM), b_fc=n(DFF), w_proj2=n(DM, DFF), b_proj2=n(DM))
              for _ in range(shape["n_layers"])]
    return dict(wte=n(NV, DM), wpe=n(CTX, DM), lnf_g=g(DM), lnf_b=n(DM), layers=layers)


def dequantized(w):
    W, mic, ts, _ = ol.quantize(w)
    return np.ascontiguousarray(ol.dequant_micro(W, mic, ts)[:, :w.shape[1]])


class OracleGpt2:
    def __init__(self, shape, wt, cap):
        self.shape, self.cap = shape, cap
        NL, DM, NH = shape["n_layers"], shape["d_model"], shape["n_heads"]
        self.t = [wt["wte"], wt["wpe"], wt["lnf_g"], wt["lnf_b"], dequantized(wt["wte"])]
        for lw in wt["layers"]:
            self.t += [dequantized(lw[k]) if k.startswith("w_") else lw[k] for k in LAYER_KEYS]
        self.t = [np.ascontiguousarray(a, np.float32) for a in self.t]
        self.ptrs = (C.c_void_p * len(self.t))(*[a.ctypes.data for a in self.t])
        self.dims = np.array([NL, DM, NH, shape["d_ff"], shape["vocab"]], np.int32)
        self.kc = np.zeros(NL * DM * cap, np.float32); self.vc = np.zeros(NL * DM * cap, np.float32)
        self.fn = ol.oracle().orc_gpt2_decode
        self.fn.restype = C.c_int
        self.fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]

    def decode(self, tok, pos):
        lg = np.zeros(self.shape["vocab"], np.float32)
        assert self.fn(self.dims.ctypes.data, self.ptrs, self.kc.ctypes.data, self.vc.ctypes.data, self.cap, int(tok), int(pos), lg.ctypes.data) == 0
        return lg


@pytest.mark.parametrize("shape,seed", [(dict(n_layers=2, d_model=128, n_heads=4, d_ff=512, vocab=300, max_ctx=64), 1),
                                        (dict(n_layers=3, d_model=192, n_heads=3, d_ff=768, vocab=1001, max_ctx=48), 2)])
def test_gpt2_teacher_forced_and_greedy(shape, seed):
    wt = synth(shape, seed)
    om = OracleGpt2(shape, wt, 48)
    gm = hb.Model.gpt2(shape, wt, kv_cap=48)
    assert gm.engine() == "graph"
    ids = np.random.default_rng(9).integers(0, shape["vocab"], 20)
    for pos, t in enumerate(ids):
        lo = om.decode(int(t), pos)
        nx, lg = gm.decode_step(int(t), pos, want_logits=True)
        assert np.max(np.abs(lo - lg)) < 2e-4, pos
        assert nx == int(np.argmax(lg)) == int(np.argmax(lo))
    # free-running greedy continuation (config 2: prompt, then new tokens)
    tok, want = int(nx), []
    for i in range(12):
        tok = int(np.argmax(om.decode(tok, 20 + i))); want.append(tok)
    got, _ = gm.decode_loop(int(nx), 20, 12)
    assert list(got) == want
    gm.close()
