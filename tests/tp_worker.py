"""One rank of the tensor-parallel decode test (launched by tests/test_tp_gpu.py through torch.distributed.run).

Every rank loads its shard of the same HXGW v3 file, the ranks exchange their 64-byte buffer handles over gloo,
then decode teacher-forced and free-running; rank 0 compares the gathered logits slices and the tokens with the
CPU restatement of the full model."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
import helix_b200 as hb                      # noqa: E402
from helix_b200.lib import check, lib       # noqa: E402


def main():
    path, n_teacher, n_free = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    check(lib().hx_set_device(int(os.environ.get("LOCAL_RANK", rank))))
    gm = hb.Model.load(path, kv_cap=256, tp_rank=rank, tp_size=world)
    mine = torch.tensor(list(gm.tp_handle()), dtype=torch.uint8)
    allh = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(allh, mine)
    gm.tp_connect([bytes(h.tolist()) for h in allh])
    dist.barrier()

    om = None
    if rank == 0:
        import oracle_lib as ol
        om = ol.OracleModel(path, kv_cap=256)
    NVl = gm.cfg.vocab
    # batched prefill inside the group: chunks of 64 positions with the partial rows of o_proj / down_proj exchanged per
    # chunk, the last position through the decode kernel; 150 tokens = two full chunks, a ragged one and the last token
    pids = np.random.default_rng(8).integers(0, NVl * world, 150).astype(np.int32)
    nxp, lgp = gm.prefill(pids, want_logits=True)
    parts = [torch.zeros(NVl, dtype=torch.float32) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(lgp.copy()))
    pf_err = 0.0
    if rank == 0:
        full = torch.cat(parts).numpy()
        lo = om.prefill(pids)
        pf_err = float(np.max(np.abs(full - lo)))
        assert pf_err < 2e-4, pf_err
        assert nxp == int(np.argmax(lo)), (nxp, int(np.argmax(lo)))
        om.reset() if hasattr(om, "reset") else None
    dist.barrier()          # rank 0 was busy with the checker: nobody starts a step (a bounded wait) before it is back
    gm.reset()
    ids = np.random.default_rng(5).integers(0, NVl * world, n_teacher)
    worst = 0.0
    for pos, t in enumerate(ids):
        nx, lg = gm.decode_step(int(t), pos, want_logits=True)
        parts = [torch.zeros(NVl, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(lg.copy()))
        nxs = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(nxs, torch.tensor([nx], dtype=torch.int64))
        assert all(int(v) == nx for v in nxs), "ranks disagree on the next token"
        if rank == 0:
            full = torch.cat(parts).numpy()
            lo = om.decode(int(t), pos)
            worst = max(worst, float(np.max(np.abs(full - lo))))
            assert nx == int(np.argmax(full)), (pos, nx, int(np.argmax(full)))
    # free-running greedy continuation on top of the cache
    out, _ = gm.decode_loop(int(ids[-1]), n_teacher - 1, n_free)
    if rank == 0:
        want = []
        tok = int(ids[-1])
        for i in range(n_free):
            tok = int(np.argmax(om.decode(tok, n_teacher - 1 + i)))
            want.append(tok)
        assert worst < 2e-4, worst
        assert list(out) == want, (list(out), want)
        print("TP-OK world=%d max-abs-logit-diff=%.3g prefill-max-abs=%.3g" % (world, worst, pf_err), flush=True)
    dist.barrier()
    gm.close()

    # a batch of three sequences inside the group: prompts of different lengths into their own KV slots, then batched
    # decode steps; the arg-max over the ranks' vocabulary slices is taken per sequence
    gb = hb.Model.load(path, kv_cap=256, tp_rank=rank, tp_size=world, batch=3)
    mine = torch.tensor(list(gb.tp_handle()), dtype=torch.uint8)
    allh = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(allh, mine)
    gb.tp_connect([bytes(h.tolist()) for h in allh])
    dist.barrier()
    rngb = np.random.default_rng(31)
    prompts = [rngb.integers(0, NVl * world, n).astype(np.int32) for n in (5, 81, 20)]
    toks = np.array([gb.prefill_seq(i, p) for i, p in enumerate(prompts)], np.int32)
    pos = np.array([len(p) for p in prompts], np.int32)
    got = [toks.copy()]
    for step in range(6):
        toks = gb.decode_batch(toks, pos + step)
        got.append(toks.copy())
    got = np.stack(got, 1)                                   # [sequence][7 tokens]
    if rank == 0:
        for i, p in enumerate(prompts):
            om.reset()
            want = om.generate(p, 7)
            assert list(got[i]) == [int(t) for t in want], (i, list(got[i]), list(want))
        print("TP-BATCH-OK world=%d" % world, flush=True)
    dist.barrier()
    gb.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
