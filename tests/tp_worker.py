"""One rank of the tensor-parallel parity run (launched by test_gpu_tp.py through torch.distributed.run).

Every rank builds the same seeded model as rank `RANK` of `WORLD_SIZE`, connects, and makes the same
calls; rank 0 also builds the single-GPU model and compares logits and greedy streams.  Prints one JSON
line on rank 0; exits non-zero on any mismatch."""
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
    from cera_b200 import synth, tp
    report = {"world": world, "cases": []}
    ok = True
    for name, cfg in CASES.items():
        cfg = dict(cfg, n_kv_heads=world, n_heads=4 * world)  # one KV head and one group of four per rank
        for kv_f16 in (0, 1):
            m = synth.build_llama(cfg, seed=11, max_seq_len=96, kv_f16=kv_f16, device=local, tp=(rank, world))
            tp.connect(m)
            prompt = synth.prompt_tokens(12, cfg["vocab_size"], seed=5)
            logits = [m.forward(int(t), pos) for pos, t in enumerate(prompt[:4])]
            last = m.forward_prefill(prompt[4:], 4)
            first = int(np.argmax(last))
            steps = [m.forward_greedy(first, 12)]
            stream, ms = m.generate_greedy(steps[0], 13, 40)
            # a prompt long enough for the batched tensor-parallel path (row-split GEMMs, column slices gathered into
            # the peers' chunk buffers), continuing from position 53
            long_prompt = synth.prompt_tokens(80, cfg["vocab_size"], seed=9)
            m.truncate_kv(0)
            batched = m.forward_prefill(long_prompt, 0)
            after = m.forward(int(np.argmax(batched)), 80)
            m.close()
            dist.barrier()
            if rank == 0:
                s = synth.build_llama(cfg, seed=11, max_seq_len=96, kv_f16=kv_f16, device=local)
                logits_1 = [s.forward(int(t), pos) for pos, t in enumerate(prompt[:4])]
                # the same per-token arithmetic as the tensor-parallel prefill
                for i, t in enumerate(prompt[4:]):
                    last_1 = s.forward(int(t), 4 + i)
                steps_1 = [s.forward_greedy(int(np.argmax(last_1)), 12)]
                stream_1, _ = s.generate_greedy(steps_1[0], 13, 40)
                s.truncate_kv(0)
                for i, t in enumerate(long_prompt):
                    per_token = s.forward(int(t), i)
                after_1 = s.forward(int(np.argmax(batched)), 80)
                s.close()

                def cosine(a, b):
                    return float(np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b)))

                # batched against per-token arithmetic: the reference's batched-prompt test holds tiled-attention paths to a
                # cosine floor of 0.99 (cera/tests/llama_batched_prefill_parity.rs); measured here 0.9999 (f16 KV 0.99989)
                cos_b, cos_a = cosine(batched, per_token), cosine(after, after_1)
                diff = max(float(np.abs(a - b).max()) for a, b in zip(logits + [last], logits_1 + [last_1]))
                scale = max(float(np.abs(b).max()) for b in logits_1)
                case_ok = (diff <= 1e-3 * scale and steps == steps_1 and list(stream) == list(stream_1) and cos_b >= 0.999 and
                           cos_a >= 0.999)
                report["cases"].append({"model": name, "kv_f16": kv_f16, "max_logit_diff": diff, "logit_scale": scale,
                                        "batched_prompt_cosine": cos_b, "decode_after_batched_prompt_cosine": cos_a,
                                        "bit_identical": diff == 0.0, "stream_equal": list(stream) == list(stream_1),
                                        "ms_per_step": ms / 40})
                ok = ok and case_ok
            dist.barrier()
    flag = torch.tensor([1 if ok else 0])
    dist.broadcast(flag, 0)
    if rank == 0:
        print(json.dumps(report), flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) else 1)


CASES = {
    # every projection on the lane-task GEMV kernel (k >= 1024)
    "wide": dict(n_layers=2, hidden_size=1024, intermediate_size=2048, n_heads=8, n_kv_heads=2, head_dim=128,
                 vocab_size=1024, rope_theta=500000.0, rms_norm_eps=1e-5, rope_type=0),
    # small extents: item-wise GEMV kernel, slices that are not multiples of 16 bytes
    "small": dict(n_layers=3, hidden_size=256, intermediate_size=512, n_heads=4, n_kv_heads=2, head_dim=64,
                  vocab_size=512, rope_theta=500000.0, rms_norm_eps=1e-5, rope_type=0),
}

if __name__ == "__main__":
    main()
