/* ref_wrap.c -- exposes the UNMODIFIED reference quantizer to the test suite.
 *
 * TEST INFRASTRUCTURE ONLY.  The reference's helixc/runtime/gpt2_pack.c is compiled where it lies
 * (its directory is given with -I by oracle/Makefile, nothing is copied); its `main` is renamed so
 * the file can be linked into a shared object, and its static functions are re-exported under
 * ref_* names.  The build keeps the reference's own flags (plain -O2, no -march, no fast-math) so
 * every float operation rounds as in the shipped importer.
 */
#define main gpt2_pack_main
#include "gpt2_pack.c"
#undef main

#define REF_API __attribute__((visibility("default")))

REF_API int   ref_e2m1_encode(float v)      { return e2m1_encode(v); }
REF_API int   ref_e2m1_encode_ref(float v)  { return e2m1_encode_ref(v); }
REF_API float ref_e2m1_decode(int c)        { return e2m1_decode(c); }
REF_API int   ref_e4m3_encode(float v)      { return e4m3_encode(v); }
REF_API float ref_e4m3_decode(int c)        { return e4m3_decode(c); }
REF_API int   ref_nvfp4_quantize(const float* w, int rows, int K, int32_t* outW, float* outSc,
                                 uint8_t* outMicro, float* outTs) {
    return nvfp4_quantize_tensor(w, rows, K, outW, outSc, outMicro, outTs);
}
REF_API void  ref_nvfp4_host_dequant(const int32_t* w, const float* sc, float* out, int rows, int Kpad) {
    nvfp4_host_dequant(w, sc, out, rows, Kpad);
}
REF_API int   ref_e2m1_equiv_selftest(void) { return e2m1_equiv_selftest(); }
REF_API int   ref_nvfp4_selftest(void)      { return nvfp4_selftest(); }
