"""Writes tests/golden/llama8b_stream.json: the greedy token stream of the CPU oracle on the benchmark's
model - the Llama-3-8B-shape random-init model (Q4_K attention / gate / up / token_embd, Q6_K ffn_down and
output, seed 0), a 512-token prompt of hashed uniform ids (seed 7) processed one token at a time, then greedy
decoding - with, per decoded token, the winning logit and the runner-up (id and value), so that a fork can be
classified with the reference's near-tie rule.  Host only (about 5 GB of weights, a few minutes on 8 cores):

    python tests/golden/make_llama8b_stream.py [--decode 288] [--threads 8]
"""
import argparse
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as O  # noqa: E402

MODEL_SEED, PROMPT_SEED, PROMPT_LEN = 0, 7, 512


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--decode", type=int, default=288)
    ap.add_argument("--threads", type=int, default=os.cpu_count() or 1)
    ap.add_argument("--out", default=os.path.join(HERE, "llama8b_stream.json"))
    args = ap.parse_args()
    t0 = time.time()
    cfg = dict(O.LLAMA3_8B)
    model = O.build_oracle_llama(cfg, seed=MODEL_SEED, max_seq_len=PROMPT_LEN + args.decode + 1, threads=args.threads)
    print(f"model built in {time.time() - t0:.1f} s", flush=True)
    prompt = O.prompt_tokens(PROMPT_LEN, cfg["vocab_size"], PROMPT_SEED)
    t0 = time.time()
    logits = None
    for pos, tok in enumerate(prompt):
        logits = model.forward(int(tok), pos, want_logits=pos == PROMPT_LEN - 1)
    print(f"prompt in {time.time() - t0:.1f} s", flush=True)

    def pick(lg):
        top = int(O.argmax(lg))
        rest = lg.copy()
        rest[top] = -np.inf
        second = int(np.argmax(rest))
        spread8 = float(np.sort(lg)[-8:][-1] - np.sort(lg)[-8:][0])
        return top, float(lg[top]), second, float(lg[second]), spread8

    first = pick(logits)
    stream, detail = [first[0]], [first]
    t0 = time.time()
    for i in range(args.decode - 1):
        logits = model.forward(stream[-1], PROMPT_LEN + i)
        p = pick(logits)
        stream.append(p[0])
        detail.append(p)
    print(f"{args.decode} tokens in {time.time() - t0:.1f} s", flush=True)
    gaps = [d[1] - d[3] for d in detail]
    out = {
        "what": "greedy stream of the CPU oracle (x86 int8 tier arithmetic, per-token prompt processing)",
        "model": "LLAMA3_8B synthetic, sigma 0.02", "model_seed": MODEL_SEED, "prompt_seed": PROMPT_SEED,
        "prompt_len": PROMPT_LEN, "kv_dtype": "f32",
        "stream": stream,  # stream[0] = pick after the prompt, stream[i] = pick after feeding stream[i-1] at position 512+i-1
        "top1_logit": [d[1] for d in detail], "top2_id": [d[2] for d in detail], "top2_logit": [d[3] for d in detail],
        "top8_spread": [d[4] for d in detail],
        "min_top2_gap": min(gaps), "min_top2_gap_at": int(np.argmin(gaps)),
    }
    with open(args.out, "w") as f:
        json.dump(out, f)
    print(f"wrote {args.out}: min top-2 gap {min(gaps):.3e} at step {int(np.argmin(gaps))}")


if __name__ == "__main__":
    main()
