"""One rank of the expert-parallel routed-FFN parity run (launched by test_gpu_tp.py through
torch.distributed.run).  Every rank owns n_expert / WORLD_SIZE experts and a ragged share of the
tokens; rank 0 also runs the single-GPU layer over all tokens.  Each rank's output rows must equal the
single-GPU rows bit for bit.  Prints one JSON line on rank 0; exits non-zero on any mismatch."""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    import cera_b200 as cb
    from cera_b200 import tp
    report = {"world": world, "cases": []}
    ok = True
    for name, (t, E, used, hs, ff, n_total) in CASES.items():
        t = getattr(cb, t)
        q = lambda n, seed: cb.quantize_weights(t, cb.synth_normal(n, seed=seed, sigma=0.02))
        gate, up, down = q(E * ff * hs, 1), q(E * ff * hs, 2), q(E * hs * ff, 3)
        router = cb.synth_normal(E * hs, seed=4, sigma=0.05)
        bias = cb.synth_normal(E, seed=6, sigma=0.2)
        x = cb.synth_normal(n_total * hs, seed=5, sigma=1.0).view(n_total, hs)
        # ragged shares: rank r takes tokens [cut[r], cut[r+1]); the last rank of a 3+ rank job gets none
        cut = [0] + [min(n_total, (r + 1) * (n_total // world) + (5 if r == 0 else 0)) for r in range(world - 1)] + [n_total]
        if world > 2:
            cut[-2] = n_total
        mine = x[cut[rank]:cut[rank + 1]]
        moe = cb.MoeFfn(E, used, hs, ff, t, gate, up, down, router, exp_probs_b=bias, max_tokens=max(1, n_total),
                        ep=(rank, world), max_total_tokens=n_total)
        tp.connect(moe)
        outs = []
        for _ in range(3):  # repeated calls reuse counters, cursors and flags
            out = moe(mine) if mine.shape[0] else moe(torch.empty(0, hs, device="cuda"))
            torch.cuda.synchronize()
            moe.check_status()
            outs.append(out.cpu().numpy())
        dist.barrier()
        gathered = [None] * world
        dist.all_gather_object(gathered, outs[-1])
        if rank == 0:
            single = cb.MoeFfn(E, used, hs, ff, t, gate, up, down, router, exp_probs_b=bias, max_tokens=n_total)
            want = single(x).cpu().numpy()
            single.close()
            got = np.concatenate([g.reshape(-1, hs) for g in gathered], axis=0)
            same = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
            stable = all(np.array_equal(outs[0], o) for o in outs)
            report["cases"].append({"case": name, "bit_identical": same, "repeatable": stable, "shares": [b - a for a, b in zip(cut, cut[1:])]})
            ok = ok and same and stable
        moe.close()
        dist.barrier()
    # More tokens than the layer was created for: every rank passes its full max_tokens while max_total_tokens is
    # the smallest value the constructor takes, so a rank's receive buffer holds exactly the average share and
    # the seeded routing's imbalance overflows at least one of them.  The plan must notice before anything is stored
    # into a peer's receive buffer, every rank must report the named error, and the layer must not hang.
    t, E, used, hs, ff = cb.Q4_0, 8, 2, 256, 128
    q = lambda n, seed: cb.quantize_weights(t, cb.synth_normal(n, seed=seed, sigma=0.02))
    per = 16
    moe = cb.MoeFfn(E, used, hs, ff, t, q(E * ff * hs, 1), q(E * ff * hs, 2), q(E * hs * ff, 3), cb.synth_normal(E * hs, seed=4, sigma=0.05),
                    max_tokens=per, ep=(rank, world), max_total_tokens=per)
    tp.connect(moe)
    moe(cb.synth_normal(per * hs, seed=50 + rank, sigma=1.0).view(per, hs))
    torch.cuda.synchronize()
    try:
        moe.check_status()
        refused = False
    except cb.CeraCudaError as e:
        refused = e.code == 1 and "receive buffer" in str(e)
    votes = [None] * world
    dist.all_gather_object(votes, refused)
    if rank == 0:
        report["overflow_refused_on_every_rank"] = all(votes)
        ok = ok and all(votes)
    moe.close()
    dist.barrier()
    flag = torch.tensor([1 if ok else 0])
    dist.broadcast(flag, 0)
    if rank == 0:
        print(json.dumps(report), flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) else 1)


CASES = {
    "small_q4_0": ("Q4_0", 8, 2, 256, 128, 37),
    "k_quant": ("Q4_K", 8, 3, 512, 256, 21),
    "lfm2moe_shape": ("Q4_0", 32, 4, 2048, 1792, 96),
}

if __name__ == "__main__":
    main()
