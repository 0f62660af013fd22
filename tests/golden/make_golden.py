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
``q8_q5_blocks.npz``      (``--blocks8``) raw Q8_0 / Q5_0 blocks (seeded, plus edge-case scales and codes)
                          with the float32 output of ``GGUFLoader._dq8`` / ``_dq5_0``
                          (adam/loaders/gguf.py:282-288, :301-310), asserted equal to ``gguf.dequantize``;
                          and float32 rows with the bytes ``gguf.quants.quantize`` makes of them, pinning
                          ``adam_b200.gguf_blocks.quantize_q8_0`` / ``quantize_q5_0``.
``tiny.gguf``,            (``--gguf``) a small Gemma-3-shaped model file written with ``gguf.GGUFWriter``
``gguf_file.npz``         (Q4_0 layers, Q8_0 token_embd, float32 norms) and what the reference's
                          ``GGUFLoader.load`` and ``ModelConfig.from_gguf_metadata`` read from it
                          (adam/loaders/gguf.py:58-133, adam/models/engine.py:56-111): metadata, tensor
                          names, types, shapes, offsets, the data offset and the configuration.
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
    ap.add_argument("--blocks8", action="store_true", help="write q8_q5_blocks.npz only")
    ap.add_argument("--gguf", action="store_true", help="write tiny.gguf and gguf_file.npz only")
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
    if args.blocks8:
        return blocks8(gguf, T, GGUFLoader)
    if args.gguf:
        return gguf_file(gguf, T, GGUFLoader, RefModelConfig)

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


def blocks8(gguf, T, GGUFLoader):
    """Q8_0 / Q5_0: the reference loader's own decode of seeded blocks, and gguf's encoders."""
    from adam_b200 import gguf_blocks as gb
    loader = GGUFLoader.__new__(GGUFLoader)
    rng = np.random.default_rng(20240602)
    edge = [0x0000, 0x8000, 0x0001, 0x83FF, 0x7BFF, 0xFBFF, 0x3C00, 0xBC00]     # zero, -0, subnormals, largest finite, +-1
    q8 = gb.random_q8_0_blocks(rng, 16, 128).reshape(-1, 34).copy()
    q5 = gb.random_q5_0_blocks(rng, 16, 128).reshape(-1, 22).copy()
    for i, bits in enumerate(edge):
        q8[i, 0], q8[i, 1] = bits & 0xFF, bits >> 8
        q5[i, 0], q5[i, 1] = bits & 0xFF, bits >> 8
    q8[8, 2:] = 0x80; q8[9, 2:] = 0x7F; q8[10, 2:] = 0x00; q8[11, 2:] = 0xFF          # codes -128, 127, 0, -1
    q5[8, 2:] = 0x00; q5[9, 2:] = 0xFF; q5[10, 2:6] = 0xFF; q5[10, 6:] = 0x00; q5[11, 2:6] = 0x00; q5[11, 6:] = 0xFF
    q8_out = loader._dq8(q8.tobytes(), q8.shape[0] * 32)
    q5_out = loader._dq5_0(q5.tobytes(), q5.shape[0] * 32)
    for raw, out, t in ((q8, q8_out, T.Q8_0), (q5, q5_out, T.Q5_0)):
        lib = gguf.dequantize(raw.reshape(1, -1), t).reshape(-1)
        assert np.array_equal(out.view(np.uint32), lib.view(np.uint32)), t
    w = (rng.standard_normal((24, 128), dtype=np.float32) * np.float32(0.02))
    w[0, :32] = 0.0                                   # all-zero block (d == 0)
    w[1, :32] = np.float32(0.01)                      # constant block
    w[2, 5] = np.float32(-0.3)                        # negative extreme
    w[3, 7] = np.float32(0.3); w[3, 9] = np.float32(-0.3)      # tie in magnitude: the first wins
    w[4, :32] = np.float32(0.005) * (np.arange(32, dtype=np.float32) - np.float32(15.5))   # codes on .5 boundaries
    raw8 = gguf.quants.quantize(w, T.Q8_0)
    raw5 = gguf.quants.quantize(w, T.Q5_0)
    assert np.array_equal(gb.quantize_q8_0(w), raw8) and np.array_equal(gb.quantize_q5_0(w), raw5)
    np.savez_compressed(os.path.join(HERE, "q8_q5_blocks.npz"), q8_0_raw=q8, q8_0_out=q8_out, q5_0_raw=q5, q5_0_out=q5_out,
                        w=w, q8_0_enc=raw8, q5_0_enc=raw5)
    print("q8_q5_blocks.npz written")


# the model of tiny.gguf: adam_b200.synth.build_model(GGUF_FILE_CFG(), Q4_0, embd_type=Q8_0, **GGUF_FILE_BUILD)
GGUF_FILE_BUILD = dict(seed=31, tied=True)


def GGUF_FILE_CFG():
    from adam_b200.config import tiny_gemma3
    return tiny_gemma3(n_layer=2, n_embd=64, n_head=2, n_head_kv=1, head_dim=32, n_ff=128, n_vocab=96, sliding_window=16)


def write_model_gguf(path, cfg, tensors, gguf, extra_kv=None):
    """Write ``tensors`` (QTensor / float32 arrays, GGUF names) and the metadata the reference reads as a .gguf
    file with ``gguf.GGUFWriter``."""
    w = gguf.GGUFWriter(path, cfg.arch)
    w.add_name("tiny synthetic model")
    w.add_context_length(cfg.n_ctx)
    w.add_block_count(cfg.n_layer)
    w.add_embedding_length(cfg.n_embd)
    w.add_feed_forward_length(cfg.n_ff)
    w.add_head_count(cfg.n_head)
    w.add_head_count_kv(cfg.n_head_kv)
    w.add_layer_norm_rms_eps(cfg.norm_eps)
    w.add_vocab_size(cfg.n_vocab)
    w.add_sliding_window(cfg.sliding_window)
    w.add_rope_freq_base(cfg.rope_base_global)
    w.add_float32(f"{cfg.arch}.rope.local_freq_base", cfg.rope_base_local)
    w.add_key_length(cfg.head_dim)
    w.add_value_length(cfg.head_dim_kv)
    w.add_token_list([f"<t{i}>" for i in range(cfg.n_vocab)])
    w.add_token_scores([float(-i) for i in range(cfg.n_vocab)])
    w.add_bos_token_id(2)
    w.add_eos_token_id(1)
    for k, v in (extra_kv or {}).items():
        w.add_string(k, v) if isinstance(v, str) else w.add_uint32(k, v)
    for name, t in tensors.items():
        if isinstance(t, np.ndarray):
            w.add_tensor(name, np.ascontiguousarray(t, np.float32))
        else:
            w.add_tensor(name, np.ascontiguousarray(t.raw).reshape(t.rows, -1), raw_dtype=gguf.GGMLQuantizationType(t.ggml_type))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def gguf_file(gguf, T, GGUFLoader, RefModelConfig):
    """tiny.gguf and what the reference's loader and configuration reader make of it."""
    import json
    from dataclasses import asdict
    from adam_b200 import gguf_blocks as gb
    from adam_b200 import synth
    cfg = GGUF_FILE_CFG()
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, embd_type=gb.GGML_TYPE_Q8_0, **GGUF_FILE_BUILD)
    path = os.path.join(HERE, "tiny.gguf")
    write_model_gguf(path, cfg, tensors, gguf, extra_kv={"general.alignment": 32})
    ld = GGUFLoader(path, keep_tensors=False, keep_raw_blocks=False)
    with contextlib.redirect_stdout(io.StringIO()):
        ld.load(verbose=False)
        rcfg = RefModelConfig.from_gguf_metadata(ld.metadata, verbose=False)
    names = [ti.name for ti in ld.tensor_infos]
    raw0 = ld.load_tensor_raw("blk.1.ffn_down.weight")
    np.savez_compressed(
        os.path.join(HERE, "gguf_file.npz"),
        metadata_json=np.array(json.dumps(ld.metadata, sort_keys=True)),
        names=np.array(names), types=np.array([ti.dtype for ti in ld.tensor_infos], np.int64),
        offsets=np.array([ti.offset for ti in ld.tensor_infos], np.int64),
        shapes_json=np.array(json.dumps({n: list(ld.tensor_shapes[n]) for n in names})),
        data_offset=np.int64(ld._data_offset), raw_bytes=np.int64(ld.estimate_raw_bytes()), f32_bytes=np.int64(ld.estimate_f32_bytes()),
        ffn_down_1_sha256=np.frombuffer(hashlib.sha256(raw0).digest(), np.uint8),
        config_json=np.array(json.dumps({k: v for k, v in asdict(rcfg).items()}, sort_keys=True)))
    print("tiny.gguf", os.path.getsize(path), "bytes; gguf_file.npz written")


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
