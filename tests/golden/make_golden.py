#!/usr/bin/env python3
"""Generate the golden fixtures in this directory by running the UNMODIFIED
reference (krokodil-byte/adam, mounted read-only) on seeded inputs.

Run where the reference tree is available:

    python tests/golden/make_golden.py --reference <checkout of krokodil-byte/adam>
    (or set ADAM_REFERENCE_DIR)

The fixtures are small ``.npz`` files; the parity tests only read them, so the
reference tree is not needed when the tests run.  What each file pins:

``q4_dequant.npz``        raw Q4_0 / Q4_K blocks (seeded, plus edge-case scales) and the
                          float32 output of ``GGUFLoader._dq4_0`` / ``_dq4k``
                          (adam/loaders/gguf.py:290-299, :312-337); the script also asserts
                          these equal ``gguf.dequantize`` bit for bit.
``q4_0_quantize.npz``     float32 input and the bytes ``gguf.quants.quantize(.., Q4_0)``
                          produces, pinning ``adam_b200.gguf_blocks.quantize_q4_0``.
``q4map_model.npz``       output of the reference's CPU model of its Q4-map storage
                          (tests/test_q4_roundtrip.py:33-63).
``decode_tiny.npz``       greedy token ids from ``check_cpu_generation``
                          (tests/diagnostics/diag_inference.py:917-1074) for small
                          Gemma-3-shaped models built by ``adam_b200.synth.build_model``
                          (tied / untied LM head, with / without QK-norm and post-norms).
``decode_1b.npz``         (only with ``--full-size``; takes several minutes and ~12 GB of RAM)
                          the same, at the full Gemma-3-1B shape of the headline benchmark:
                          26 layers, hidden 1152, vocabulary 262144, Q4_0, a 128-token prompt and
                          128 greedy tokens, tied and untied LM head.  Beside the reference's ids the
                          file records the smallest gap between the best and the second-best logit
                          along the decoded path (from the numpy restatement, whose ids must equal the
                          reference's), so a reader can see how well-conditioned the arg-max is.
"""
import argparse
import hashlib
import importlib.util
import io
import contextlib
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

# the tiny decode cases: (name, build kwargs, cfg kwargs, n_prompt, n_gen)
DECODE_CASES = [
    ("tied", dict(seed=11, tied=True), dict(), 12, 24),
    ("untied", dict(seed=12, tied=False), dict(), 9, 24),
    ("untied_noqk", dict(seed=13, tied=False, qk_norm=False, post_norms=False), dict(n_head=2, n_head_kv=2), 7, 16),
    ("gqa2", dict(seed=14, tied=False), dict(n_head=4, n_head_kv=2, head_dim=32, n_layer=7), 10, 20),
]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("ADAM_REFERENCE_DIR", ""))
    ap.add_argument("--full-size", action="store_true", help="write decode_1b.npz (1B-shape model) instead of the small fixtures")
    args = ap.parse_args()
    ref = args.reference
    if not ref or not os.path.isdir(ref):
        ap.error("give the reference checkout with --reference or ADAM_REFERENCE_DIR")
    sys.path.insert(0, os.path.join(ref, "adamah-MAIN"))
    sys.path.insert(0, ref)

    import gguf
    from gguf import GGMLQuantizationType as T
    from adam.loaders.gguf import GGUFLoader
    from adam.models.engine import ModelConfig as RefModelConfig

    from adam_b200 import gguf_blocks as gb
    from adam_b200 import synth
    from adam_b200.config import tiny_gemma3
    from dataclasses import asdict, replace

    if args.full_size:
        return full_size(ref, gguf, T, RefModelConfig)

    loader = GGUFLoader.__new__(GGUFLoader)
    rng = np.random.default_rng(20240601)

    # ---- 1. block decode ---------------------------------------------------
    q40 = gb.random_q4_0_blocks(rng, 24, 256).reshape(-1, 18).copy()
    # edge-case scales: zero, negative, subnormal, largest finite
    for i, bits in enumerate([0x0000, 0x8000, 0x0001, 0x83FF, 0x7BFF, 0xFBFF, 0x3C00, 0xBC00]):
        q40[i, 0] = bits & 0xFF
        q40[i, 1] = bits >> 8
    q40[8, 2:] = 0x00
    q40[9, 2:] = 0xFF
    q40_out = loader._dq4_0(q40.tobytes(), q40.shape[0] * 32)
    lib = gguf.dequantize(q40.reshape(1, -1), T.Q4_0).reshape(-1)
    assert np.array_equal(q40_out.view(np.uint32), lib.view(np.uint32))

    q4k = gb.random_q4_k_blocks(rng, 6, 1024).reshape(-1, 144).copy()
    for i, (db, mb) in enumerate([(0x0000, 0x0000), (0x8001, 0x0001), (0x7BFF, 0x0400), (0x3C00, 0xBC00)]):
        q4k[i, 0], q4k[i, 1] = db & 0xFF, db >> 8
        q4k[i, 2], q4k[i, 3] = mb & 0xFF, mb >> 8
    q4k[4, 4:16] = 0xFF
    q4k[5, 4:16] = 0x00
    q4k[6, 16:] = 0xFF
    q4k_out = loader._dq4k(q4k.tobytes(), q4k.shape[0] * 256)
    lib = gguf.dequantize(q4k.reshape(1, -1), T.Q4_K).reshape(-1)
    with np.errstate(invalid="ignore"):
        same = (q4k_out.view(np.uint32) == lib.view(np.uint32)) | (np.isnan(q4k_out) & np.isnan(lib))
    assert same.all()
    np.savez_compressed(os.path.join(HERE, "q4_dequant.npz"),
                        q4_0_raw=q40, q4_0_out=q40_out, q4_k_raw=q4k, q4_k_out=q4k_out)

    # ---- 2. Q4_0 encoder ---------------------------------------------------
    w = (rng.standard_normal((48, 256), dtype=np.float32) * np.float32(0.02))
    w[0, :32] = 0.0                      # all-zero block (d == 0)
    w[1, :32] = np.float32(0.01)         # constant block
    w[2, 5] = np.float32(-0.3)           # negative extreme
    w[3, 7] = np.float32(0.3); w[3, 9] = np.float32(-0.3)   # tie in magnitude: first wins
    raw = gguf.quants.quantize(w, T.Q4_0)
    np.savez_compressed(os.path.join(HERE, "q4_0_quantize.npz"), w=w, raw=raw)
    assert np.array_equal(gb.quantize_q4_0(w), raw), "adam_b200 Q4_0 encoder differs from gguf"

    # ---- 3. reference CPU model of the Q4 map --------------------------------
    spec = importlib.util.spec_from_file_location("ref_q4_roundtrip", os.path.join(ref, "tests/test_q4_roundtrip.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    data = (rng.standard_normal(32 * 40, dtype=np.float32) * np.float32(0.05))
    data[:32] = np.float32(0.25)         # flat group -> scale 1.0 branch
    scales, zeros = mod.quantize_groups(data, 32)
    deq = mod.dequantize_groups(data, scales, zeros, 32)
    np.savez_compressed(os.path.join(HERE, "q4map_model.npz"), data=data, scales=scales, zeros=zeros, deq=deq)

    # ---- 4. greedy decode ids from the unmodified numpy decoder --------------
    spec = importlib.util.spec_from_file_location("ref_diag_inference", os.path.join(ref, "tests/diagnostics/diag_inference.py"))
    diag = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(diag)
    out = {}
    for name, bkw, ckw, n_prompt, n_gen in DECODE_CASES:
        cfg = replace(tiny_gemma3(), **ckw)
        if "head_dim" in ckw:
            cfg = replace(cfg, head_dim_kv=ckw["head_dim"])
        tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, **bkw)
        h = hashlib.sha256()
        f32 = {}
        for k in sorted(tensors):
            t = tensors[k]
            if isinstance(t, np.ndarray):
                f32[k] = t
                h.update(t.tobytes())
            else:
                h.update(t.raw.tobytes())
                f32[k] = gguf.dequantize(t.raw.reshape(t.rows, -1), T.Q4_0).reshape(t.rows, t.cols)
        prompt = synth.random_prompt(cfg.n_vocab, n_prompt, seed=bkw["seed"] + 100)
        rcfg = RefModelConfig(**{k: v for k, v in asdict(cfg).items()})

        class Tok:
            eos_id = -1; bos_id = 2; _specials = {}; _vocab = None
            def encode(self, text, add_bos=True): return [int(x) for x in prompt]
            def decode(self, toks): return " ".join(map(str, toks))

        eng = types.SimpleNamespace(tensors=f32, _kv_cap=n_prompt + n_gen + 1)
        with contextlib.redirect_stdout(io.StringIO()):
            diag.check_cpu_generation(eng, Tok(), rcfg, n_tokens=n_gen)
        toks = np.array(eng._last_cpu_gen_tokens, np.int32)
        print(f"{name}: {toks.tolist()}")
        out[f"{name}_tokens"] = toks
        out[f"{name}_prompt"] = prompt
        out[f"{name}_sha256"] = np.frombuffer(h.digest(), np.uint8)
    np.savez_compressed(os.path.join(HERE, "decode_tiny.npz"), **out)
    print("fixtures written to", HERE)


# the full-size decode cases: (name, build kwargs, n_prompt, n_gen); the model is
# adam_b200.config.gemma3_1b() built by adam_b200.synth.build_model on the host
FULL_SIZE_CASES = [
    ("tied", dict(seed=21, tied=True), 128, 128),
    ("untied", dict(seed=22, tied=False), 128, 128),
]


def full_size(ref, gguf, T, RefModelConfig):
    """Greedy ids of the unmodified reference decoder at the Gemma-3-1B shape."""
    from dataclasses import asdict
    from adam_b200 import gguf_blocks as gb
    from adam_b200 import synth
    from adam_b200.config import gemma3_1b
    from oracle import cref
    from oracle.decoder import OracleDecoder

    spec = importlib.util.spec_from_file_location("ref_diag_inference", os.path.join(ref, "tests/diagnostics/diag_inference.py"))
    diag = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(diag)
    cfg = gemma3_1b()
    out = {}
    for name, bkw, n_prompt, n_gen in FULL_SIZE_CASES:
        tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, **bkw)
        h = hashlib.sha256()
        f32 = {}
        for k in sorted(tensors):
            t = tensors[k]
            if isinstance(t, np.ndarray):
                f32[k] = t
                h.update(t.tobytes())
            else:
                h.update(t.raw.tobytes())
                f32[k] = cref.dequant(t.raw, t.ggml_type, t.rows, t.cols)
        # the threaded C decode is the same bits as gguf.dequantize (spot check on one layer's matrices)
        for k in ("blk.0.attn_q.weight", "blk.0.ffn_down.weight"):
            t = tensors[k]
            lib = gguf.dequantize(t.raw.reshape(t.rows, -1), T.Q4_0).reshape(t.rows, t.cols)
            assert np.array_equal(lib.view(np.uint32), f32[k].view(np.uint32))
        del tensors
        prompt = synth.random_prompt(cfg.n_vocab, n_prompt, seed=bkw["seed"] + 100)
        rcfg = RefModelConfig(**{k: v for k, v in asdict(cfg).items()})

        class Tok:
            eos_id = -1; bos_id = 2; _specials = {}; _vocab = None
            def encode(self, text, add_bos=True): return [int(x) for x in prompt]
            def decode(self, toks): return " ".join(map(str, toks))

        eng = types.SimpleNamespace(tensors=f32, _kv_cap=n_prompt + n_gen + 1)
        with contextlib.redirect_stdout(io.StringIO()):
            diag.check_cpu_generation(eng, Tok(), rcfg, n_tokens=n_gen)
        toks = np.array(eng._last_cpu_gen_tokens, np.int32)
        # the restatement must reproduce them; it also yields the logits, hence the arg-max margins
        dec = OracleDecoder(cfg, f32, kv_cap=n_prompt + n_gen + 1)
        got, logits = dec.generate(prompt, n_gen, keep_logits=True)
        assert got == toks.tolist(), "oracle/decoder.py does not reproduce the reference's ids at full size"
        gaps = []
        for lg in logits:
            top2 = np.partition(lg, -2)[-2:]
            gaps.append(float(top2[1] - top2[0]))
        print(f"{name}: {toks.tolist()}\n  smallest top-2 logit gap along the path: {min(gaps):.3e} (largest |logit| {float(np.abs(logits[0]).max()):.3f})")
        out[f"{name}_tokens"] = toks
        out[f"{name}_prompt"] = prompt
        out[f"{name}_sha256"] = np.frombuffer(h.digest(), np.uint8)
        out[f"{name}_top2_gaps"] = np.array(gaps, np.float32)
        del f32, eng, dec
    np.savez_compressed(os.path.join(HERE, "decode_1b.npz"), **out)
    print("decode_1b.npz written to", HERE)


if __name__ == "__main__":
    main()
