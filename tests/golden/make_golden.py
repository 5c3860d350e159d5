"""Generates the committed golden fixtures from the REFERENCE's own operators
(oracle/_ref/libkdnn_ref.so, compiled from the reference's headers). Run here,
where the reference sources exist:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402
from oracle import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def gguf_fixture_tensors(gp):
    """Tensors of the container fixture: seeded, so the reader test regenerates the expected bytes."""
    return [("token_embd.weight", [256, 4], O.Q6_K, gp.random_payload(O.Q6_K, 4, 256, 901)),
            ("blk.0.ffn_gate_exps.weight", [256, 5, 3], O.Q4_K, gp.random_payload(O.Q4_K, 15, 256, 902)),
            ("blk.0.attn_q.weight", [64, 3], O.Q8_0, gp.random_payload(O.Q8_0, 3, 64, 903)),
            ("blk.1.ffn_down.weight", [512, 2], O.Q5_K, gp.random_payload(O.Q5_K, 2, 512, 904)),
            ("output_norm.weight", [7], 0, np.arange(7, dtype=np.float32) * 0.5)]


def main():
    O.build()
    ref = O.Ref()
    gp = ge._load_module("_gp", os.path.join(ge.PKG_DIR, "ggml_pack.py"))
    out = {}
    rng = np.random.default_rng(20261125)
    cases = [("q4k_f32", O.Q4_K, 9, 1024, False, "random"), ("q4k_bf16", O.Q4_K, 6, 4096, True, "synth"),
             ("q6k_f32", O.Q6_K, 9, 2048, False, "random"), ("q6k_bf16", O.Q6_K, 5, 2048, True, "synth"),
             ("q80_f32", O.Q8_0, 9, 1024, False, "random"), ("q80_bf16", O.Q8_0, 5, 512, True, "synth"),
             ("q4k_odd_f32", O.Q4_K, 3, 6656, False, "random")]
    for i, (tag, dt, rows, K, bf16, kind) in enumerate(cases):
        w = gp.random_payload(dt, rows, K, 100 + i) if kind == "random" else gp.synth_weight(dt, rows, K, 100 + i)
        x = rng.standard_normal(K).astype(np.float32)
        if bf16:
            x = O.bf16_round(x)
        y, staging = ref.quant_gemv(dt, O.aligned_copy(w), rows, K, x, bf16=bf16, int8=True)
        out[tag + "_w"] = w
        out[tag + "_x"] = x
        out[tag + "_y"] = y
        out[tag + "_staging"] = np.array(staging)
        out[tag + "_meta"] = np.array([dt, rows, K], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "gemv_int8.npz"), **out)

    # router: the fixed logits of tests/Test_MoE.cpp:71-75 plus seeded cases
    r = {}
    fixed = np.array([[0.1, 2.0, -1.0, 0.5, 1.2, -0.3], [1.5, 1.5, 1.5, -2.0, 0.0, 3.0],
                      [-0.5, -0.2, -0.8, -0.1, -1.5, -0.4]], dtype=np.float32)
    n = 0
    for lg, bias, k, norm, scale, sig, bf16 in [
            (fixed, None, 2, True, 1.0, False, False), (fixed, None, 3, False, 1.0, False, False),
            (fixed, np.array([0, 0, 5, 0, 0, 0], np.float32), 2, True, 2.5, False, False),
            (fixed, None, 2, True, 1.0, True, False), (fixed, np.array([0, 0, 5, 0, 0, 0], np.float32), 2, False, 1.0, True, False),
            (rng.standard_normal((64, 8)).astype(np.float32), None, 2, True, 1.0, False, True),
            (rng.standard_normal((256, 128)).astype(np.float32), None, 8, True, 1.0, False, True),
            (np.round(rng.standard_normal((40, 64)) * 2).astype(np.float32) / 2, None, 4, True, 1.0, False, False)]:
        if bf16:
            lg = O.bf16_round(lg)
        idx, w = ref.moe_route(lg, bias, k, norm, scale, sig, bf16=bf16)
        r[f"c{n}_logits"] = lg
        r[f"c{n}_bias"] = np.zeros(0, np.float32) if bias is None else bias
        r[f"c{n}_cfg"] = np.array([k, int(norm), int(sig), int(bf16)], dtype=np.int64)
        r[f"c{n}_scale"] = np.array([scale], dtype=np.float32)
        r[f"c{n}_idx"] = idx
        r[f"c{n}_w"] = w
        n += 1
    np.savez_compressed(os.path.join(HERE, "moe_route.npz"), **r)

    # fused one-token MoE decode of the reference (fp path), small expert shape
    m = {}
    E, H, F, S = 3, 256, 256, 2
    gate = [gp.synth_weight(O.Q4_K, F, H, 300 + e) for e in range(E)]
    up = [gp.synth_weight(O.Q4_K, F, H, 400 + e) for e in range(E)]
    down = [gp.synth_weight(O.Q4_K, H, F, 500 + e, std=0.05) for e in range(E)]
    x = O.bf16_round(rng.standard_normal(H).astype(np.float32))
    idx = np.array([2, 0], dtype=np.int32)
    wts = np.array([0.7, 0.3], dtype=np.float32)
    al = lambda lst: [O.aligned_copy(a) for a in lst]
    Y, act = ref.quant_moe_decode(x, al(gate), al(up), al(down), idx, wts, F, bf16=True)
    m.update(gate=np.stack(gate), up=np.stack(up), down=np.stack(down), x=x, idx=idx, wts=wts, Y=Y, act=act,
             meta=np.array([E, H, F, S], dtype=np.int64))
    np.savez_compressed(os.path.join(HERE, "moe_decode_fp.npz"), **m)
    # a container written by the reference's own writer (tests/test_gguf_io.py reads it back)
    ref.gguf_write(os.path.join(HERE, "ref_written.gguf"), gguf_fixture_tensors(gp),
                   strings={"general.architecture": "lfm2moe", "general.name": "fixture"},
                   f32={"lfm2moe.attention.layer_norm_rms_epsilon": 1e-5},
                   u32={"lfm2moe.block_count": 2, "lfm2moe.expert_count": 3})
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
