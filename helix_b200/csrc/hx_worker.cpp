// hx_worker -- the serve worker as a process: what a host that spawns the reference's
//   gpt2_infer <combined.ptx> <weights> --serve [--emit-fd N] [--max-ctx M] [--vocab v.json --merges m.txt]
// (helixc/runtime/gpt2_infer.c:3540-3560) spawns instead:
//   hx_worker <weights> --serve [--emit-fd N] [--max-ctx M] [--vocab v.json --merges m.txt]
// HX_SPECIALS=1 splits control tokens off prompts and HX_EOS=<id> ends a request at that token, as in the reference.
// Requests arrive on stdin, one JSON frame per line; events leave on the emit descriptor (default stdout); the
// readiness line goes to stderr like the reference's (:3303).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "../../include/helix_b200.h"

int main(int argc, char** argv) {
    if (argc < 3 || strcmp(argv[2], "--serve") != 0) {
        fprintf(stderr, "usage: %s <weights> --serve [--emit-fd N] [--max-ctx M] [--device D] [--vocab v.json --merges m.txt]\n", argv[0]);
        return 2;
    }
    int emit_fd = 1, max_ctx = 512, device = 0;
    const char *vocab = NULL, *merges = NULL;
    for (int i = 3; i < argc; i++) {
        if (!strcmp(argv[i], "--emit-fd") && i + 1 < argc) emit_fd = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--max-ctx") && i + 1 < argc) max_ctx = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--device") && i + 1 < argc) device = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--vocab") && i + 1 < argc) vocab = argv[++i];
        else if (!strcmp(argv[i], "--merges") && i + 1 < argc) merges = argv[++i];
    }
    if (hx_set_device(device) != HX_OK) { fprintf(stderr, "hx_worker: %s\n", hx_last_error()); return 2; }
    const int kv_cap = ((max_ctx + 63) / 64) * 64 < 64 ? 64 : ((max_ctx + 63) / 64) * 64;
    hx_model* m = NULL;
    if (hx_model_load(&m, argv[1], kv_cap, 1, 0, 0, 1) != HX_OK) { fprintf(stderr, "hx_worker: %s\n", hx_last_error()); return 2; }
    hx_tokenizer* tok = NULL;
    if (vocab && merges && hx_tokenizer_load(&tok, vocab, merges) != HX_OK) { fprintf(stderr, "hx_worker: %s\n", hx_last_error()); return 2; }
    const char* e;
    const int specials = (e = getenv("HX_SPECIALS")) ? atoi(e) : 0;
    const int eos = (e = getenv("HX_EOS")) ? atoi(e) : -1;
    fprintf(stderr, "GPT2_SERVE_READY\n"); fflush(stderr);
    const int rc = hx_serve_text(m, tok, specials, eos, 0, emit_fd, max_ctx);
    hx_tokenizer_free(tok);
    if (rc != HX_OK) fprintf(stderr, "hx_worker: %s\n", hx_last_error());
    hx_model_free(m);
    return rc == HX_OK ? 0 : 1;
}
