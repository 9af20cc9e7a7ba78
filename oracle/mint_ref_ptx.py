#!/usr/bin/env python
"""Mints the reference's own GPU kernels (PTX) from the reference tree, for the checker.

TEST INFRASTRUCTURE ONLY: nothing in the shipped library reads these files.  The reference worker
(helixc/runtime/gpt2_infer.c) loads PTX that the Helix compiler `kovc` emits from the kernel sources
under helixc/examples/.  This script rebuilds that chain with gcc, from the sources where they lie
(nothing is copied into this repository; all outputs go to oracle/_ref/, which is not tracked):

  1. the frozen C seed (stage0/helixc-bootstrap/seed.c) is compiled with gcc, exactly as
     stage0/helixc-bootstrap/ddc_fixpoint_gcc.sh:9-15 does;
  2. the K1 PTX driver source is assembled the way stage0/helixc-bootstrap/assemble_k1.hx does:
     strip_demo(lexer.hx) + parser.hx + strip_demo(kovc.hx) + drivers/driver_k1ptxdrv.hx, CRs removed
     (the driver's two fixed file names are redirected into the output folder);
  3. the seed compiles that source into the kovc PTX driver;
  4. the driver emits
       model14.ptx        the 14-kernel module of scripts/llama_model_gate.sh:72
       <kernel>.ptx       the side modules the worker loads through HX_DQPTX, HX_FUSEDGEMV_PTX,
                          HX_GEMV3_PTX, HX_FUSEDATTN_PTX and HX_SPEC_PTX.
  Every kernel that has a committed `.ref.ptx` next to its source is compared with it byte for byte.

usage: python oracle/mint_ref_ptx.py <path to the Helix tree> [<output folder>]
"""
import os
import subprocess
import sys

MODEL14 = ["tiled_matmul", "tiled_matmul_abt", "gpu_softmax_causal", "gpu_layernorm_fwd_eps", "gpu_add_bias_rowbcast",
           "gpu_gelu_stable", "vector_add", "gpu_scale_rt", "gpu_rmsnorm_fwd_eps", "gpu_rope_rot", "gpu_silu_mul",
           "gpu_gemv_abt", "gpu_gemv_ab", "gpu_softmax_row"]
SIDE = ["nvfp4_dequant_tiled", "dequant_gemv_blockred", "dequant_gemv_warp", "fused_decode_attn", "softmax_causal_offset"]
INC = ["-include", "stdio.h", "-include", "stdlib.h", "-include", "unistd.h", "-include", "string.h"]


def strip_demo(raw):
    """Everything before the dashes line that precedes '// Demo:' (offsets taken on the raw bytes)."""
    i = raw.find(b"\n// Demo:")
    if i < 0:
        raise SystemExit("no '// Demo:' marker")
    j = raw.rfind(b"\n", 0, i)
    return raw[:j + 1]


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    ref = os.path.abspath(sys.argv[1])
    out = os.path.abspath(sys.argv[2]) if len(sys.argv) > 2 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "kovc")
    os.makedirs(out, exist_ok=True)
    boot, ex = os.path.join(ref, "helixc", "bootstrap"), os.path.join(ref, "helixc", "examples")
    s0 = os.path.join(ref, "stage0", "helixc-bootstrap")
    seed = os.path.join(out, "seed_gcc")
    subprocess.check_call(["gcc", "-std=gnu89", "-w", *INC, "-o", seed, os.path.join(s0, "seed.c")])
    rd = lambda p: open(p, "rb").read()
    src = (strip_demo(rd(os.path.join(boot, "lexer.hx"))) + rd(os.path.join(boot, "parser.hx")) +
           strip_demo(rd(os.path.join(boot, "kovc.hx"))) + rd(os.path.join(s0, "drivers", "driver_k1ptxdrv.hx"))).replace(b"\r", b"")
    src = src.replace(b'"/tmp/kernel_in.hx"', b'"kernel_in.hx"').replace(b'"/tmp/out.ptx"', b'"out.ptx"')
    open(os.path.join(out, "k1ptxdrv.hx"), "wb").write(src)
    drv = os.path.join(out, "kovc_ptxdrv.bin")
    subprocess.check_call([seed, "k1ptxdrv.hx", "kovc_ptxdrv.bin"], cwd=out)
    os.chmod(drv, 0o755)

    def emit(kernels, name):
        text = b"".join(rd(os.path.join(ex, k + "_kernel.hx")).replace(b"\r", b"") + b"\n" for k in kernels)
        open(os.path.join(out, "kernel_in.hx"), "wb").write(text)
        tmp = os.path.join(out, "out.ptx")
        if os.path.exists(tmp):
            os.remove(tmp)
        subprocess.call(["bash", "-c", "ulimit -s unlimited; exec ./kovc_ptxdrv.bin"], cwd=out,
                        stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        if not os.path.exists(tmp) or os.path.getsize(tmp) == 0:
            raise SystemExit(f"kovc emitted nothing for {name}")
        ptx = rd(tmp)
        open(os.path.join(out, name + ".ptx"), "wb").write(ptx)
        return ptx

    m = emit(MODEL14, "model14")
    missing = [k for k in MODEL14 if (".entry " + k).encode() not in m]
    if missing:
        raise SystemExit(f"model14.ptx lacks entries {missing}")
    same = 0
    for k in SIDE + ["tiled_matmul", "vector_add"]:
        p = emit([k], k)
        refp = os.path.join(ex, k + "_kernel.ref.ptx")
        if os.path.exists(refp):
            if rd(refp).replace(b"\r", b"") != p:
                raise SystemExit(f"{k}: emitted PTX differs from the committed {os.path.basename(refp)}")
            same += 1
    print(f"kovc minted; model14.ptx {len(m)} bytes, {len(SIDE)} side modules, {same} byte-identical to the committed .ref.ptx")


if __name__ == "__main__":
    main()
