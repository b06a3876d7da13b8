"""What each departure from the reference's rounding points costs, oracle against oracle (CPU only, no GPU).

Runs the Qwen3-0.6B-shaped random-init model of the decode parity test at a given depth through tests/oracle_model.py
once as the reference does it and once per listed deviation (see OracleModel: kv_unrounded, ffn_unrounded, no_split,
act_q16, act_q24, sum_order, prefill_matvec; `flipP` flips the lowest fp16 bit of a fraction P of the activations
entering every layer; `a+b` combines deviations), teacher-forced with the reference run's greedy tokens, and prints
max |dlogit| and top-1 agreement per deviation.

    python -m tests.rounding_ablation <layers> <prompt tokens> <steps> <dev,dev,...>

Measured (prompt 64, 32 steps; max |dlogit| / top-1 agreement):

    deviation                              4 layers      8 layers      16 layers     28 layers
    kv_unrounded                           0.0078/1.00   0.0068/1.00   0.0063/1.00   0.0071/1.00
    ffn_unrounded                          0.0079/1.00   0.0078/1.00   0.0068/1.00   0.0078/1.00
    act_q16                                0.0272/0.94   0.0142/1.00   0.0083/1.00   0.0095/1.00
    act_q24                                0.0076/1.00   0.0078/1.00   0.0065/1.00   0.0073/1.00
    kv_unrounded+ffn_unrounded+act_q16     0.0288/0.94   0.0156/1.00   0.0081/1.00   0.0092/1.00
    sum_order                              0.0288/0.94   0.0381/1.00   0.0486/0.94   0.0566/0.88
    prefill_matvec                         0.0649/0.94   0.0713/0.94   0.0743/0.97   0.0878/0.94
    flip0.002                              0.0381/0.94   0.0518/0.97   0.0561/1.00   0.0762/0.88
    flip0.02                               0.0508/0.91   0.0605/0.94   0.0723/1.00   0.0862/0.97
"""
import json
import sys
import time

import numpy as np

from ironmill_b200.bundle import ModelConfig
from oracle import oracle as orc
from tests import helpers as H
from tests.oracle_model import OracleModel, synth_model


def main(argv):
    L, prompt_len, steps = int(argv[1]), int(argv[2]), int(argv[3])
    devs = argv[4].split(",") if len(argv) > 4 else []
    cfg = ModelConfig(architecture="qwen3", hidden_size=1024, intermediate_size=3072, num_hidden_layers=L, num_attention_heads=16,
                      num_key_value_heads=8, head_dim=128, vocab_size=151936, max_position_embeddings=4096, rms_norm_eps=1e-6,
                      rope_theta=1e6, tie_word_embeddings=False)
    tensors = synth_model(cfg, seed=3)
    tqc = orc.TqConstants(128, 8, seed=42)
    max_seq = prompt_len + steps + 8
    ref = OracleModel(cfg, tensors, tqc, max_seq)
    variants = {}
    for d in devs:
        if d.startswith("flip"):
            variants[d] = OracleModel(cfg, tensors, tqc, max_seq, flip_rate=float(d[4:]))
        else:
            variants[d] = OracleModel(cfg, tensors, tqc, max_seq, deviations=d.split("+"))
    prompt = H.rng_for("prompt").integers(0, cfg.vocab_size, prompt_len).astype(np.uint32)
    t0 = time.time()
    r = ref.forward(prompt)
    for m in variants.values():
        m.forward(prompt)
    err = {d: [] for d in variants}
    agree = {d: [] for d in variants}
    for _ in range(steps):
        tok = orc.argmax(r)
        r = ref.forward([tok])
        for d, m in variants.items():
            o = m.forward([tok])
            err[d].append(float(np.abs(o - r).max()))
            agree[d].append(int(orc.argmax(o) == orc.argmax(r)))
    for d in variants:
        print(json.dumps({"layers": L, "deviation": d, "max_abs_dlogit": max(err[d]), "top1": float(np.mean(agree[d]))}))
    print(f"# {time.time() - t0:.0f} s", file=sys.stderr)


if __name__ == "__main__":
    main(sys.argv)
