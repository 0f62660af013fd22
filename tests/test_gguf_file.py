"""The GGUF file reader against what the UNMODIFIED reference reads from the same file
(tests/golden/tiny.gguf and gguf_file.npz, written by tests/golden/make_golden.py --gguf from
adam/loaders/gguf.py:58-133 and adam/models/engine.py:56-111), against the ``gguf`` package's own
reader, and -- when a checkout of the reference is at hand -- against the reference run live.  CPU only."""
import hashlib
import json
import os
import sys

import numpy as np
import pytest

from adam_b200 import gguf_blocks as gb
from adam_b200 import synth
from adam_b200.config import ModelConfig
from adam_b200.gguf_file import GGUFLoader, QUANT_INFO

from tests.golden.make_golden import GGUF_FILE_BUILD, GGUF_FILE_CFG, write_model_gguf

REFERENCE = os.environ.get("ADAM_REFERENCE_DIR", "/root/reference")


@pytest.fixture()
def tiny(golden_dir):
    ld = GGUFLoader(os.path.join(golden_dir, "tiny.gguf")).load()
    yield ld, np.load(os.path.join(golden_dir, "gguf_file.npz"))
    ld.close()


def test_header_metadata_and_tensor_table(tiny):
    ld, g = tiny
    want_meta = json.loads(str(g["metadata_json"]))
    assert json.loads(json.dumps(ld.metadata, sort_keys=True)) == want_meta
    assert [ti.name for ti in ld.tensor_infos] == g["names"].tolist()
    assert [ti.dtype for ti in ld.tensor_infos] == g["types"].tolist()
    assert [ti.offset for ti in ld.tensor_infos] == g["offsets"].tolist()
    assert {n: list(s) for n, s in ld.tensor_shapes.items()} == json.loads(str(g["shapes_json"]))
    assert ld._data_offset == int(g["data_offset"])
    assert ld.estimate_raw_bytes() == int(g["raw_bytes"]) and ld.estimate_f32_bytes() == int(g["f32_bytes"])
    assert ld.get_bos_token_id() == 2 and ld.get_eos_token_id() == 1 and len(ld.get_tokenizer_vocab()) == 96
    assert ld.tensor_types["token_embd.weight"] == 8 and ld.tensor_types["blk.0.attn_q.weight"] == 2


def test_raw_blocks_are_the_files_bytes(tiny):
    ld, g = tiny
    raw = ld.load_tensor_raw("blk.1.ffn_down.weight")
    assert np.array_equal(np.frombuffer(hashlib.sha256(raw.tobytes()).digest(), np.uint8), g["ffn_down_1_sha256"])
    # the file holds exactly the model it was written from
    tensors = synth.build_model(GGUF_FILE_CFG(), gb.GGML_TYPE_Q4_0, embd_type=gb.GGML_TYPE_Q8_0, **GGUF_FILE_BUILD)
    got = ld.model_tensors()
    assert sorted(got) == sorted(tensors)
    for name, t in tensors.items():
        if isinstance(t, np.ndarray):
            assert np.array_equal(got[name].reshape(-1), t.reshape(-1))
        else:
            q = got[name]
            assert (q.ggml_type, q.rows, q.cols) == (t.ggml_type, t.rows, t.cols) and np.array_equal(q.raw, t.raw)
            off, n = ld.tensor_file_range(name)
            assert q.file == (str(ld.path), off) and n == t.raw.size
    # chunks cover the tensor in whole blocks, in order
    parts = list(ld.iter_tensor_chunks("token_embd.weight", max_chunk_mb=1))
    assert sum(p[1] for p in parts) == 96 * 64 and np.array_equal(np.concatenate([p[2] for p in parts]), tensors["token_embd.weight"].raw)
    with pytest.raises(NotImplementedError):
        ld.load_tensor_f32("token_embd.weight")       # quantized blocks are decoded on the device only
    del got, q, raw, parts


def test_config_from_metadata_and_shapes(tiny):
    ld, g = tiny
    want = json.loads(str(g["config_json"]))
    got = ModelConfig.from_gguf_metadata(ld.metadata)
    for k, v in want.items():
        assert getattr(got, k) == pytest.approx(v), k
    # after the shape pass the configuration is the one the file was written from
    cfg, src = ld.model_config(), GGUF_FILE_CFG()
    for k in ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "head_dim_kv", "n_ff", "n_vocab", "sliding_window", "ffn_act",
              "rope_base_global", "rope_base_local", "attn_softcap", "final_softcap", "norm_eps"):
        assert getattr(cfg, k) == pytest.approx(getattr(src, k)), k
    assert cfg.emb_scale == pytest.approx(src.emb_scale)


def test_against_the_gguf_package_reader(tmp_path):
    """A second file (Q4_K layers, Q5_0 token_embd, untied head) read by this reader and by gguf.GGUFReader."""
    gguf = pytest.importorskip("gguf")
    from adam_b200.config import tiny_gemma3
    cfg = tiny_gemma3(n_layer=1, n_embd=256, n_head=4, n_head_kv=1, head_dim=64, n_ff=256, n_vocab=64)
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_K, seed=5, tied=False, embd_type=gb.GGML_TYPE_Q5_0)
    path = str(tmp_path / "m.gguf")
    write_model_gguf(path, cfg, tensors, gguf)
    ld = GGUFLoader(path).load()
    rd = gguf.GGUFReader(path)
    assert [t.name for t in rd.tensors] == [ti.name for ti in ld.tensor_infos]
    for t in rd.tensors:
        ti = ld.get_tensor_info(t.name)
        assert int(t.tensor_type) == ti.dtype and [int(x) for x in t.shape] == list(ti.shape)
        assert int(t.data_offset) == ld.tensor_file_range(t.name)[0] and int(t.n_bytes) == ld.tensor_file_range(t.name)[1]
        assert np.array_equal(np.asarray(t.data).reshape(-1).view(np.uint8), ld.load_tensor_raw(t.name))
    assert ld.metadata["gemma3.block_count"] == 1 and ld.metadata["general.architecture"] == "gemma3"
    del rd
    ld.close()


def test_bad_files_are_refused(tmp_path, golden_dir):
    data = open(os.path.join(golden_dir, "tiny.gguf"), "rb").read()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUX" + data[4:])
    with pytest.raises(ValueError, match="Bad magic"):
        GGUFLoader(str(bad)).load()
    short = tmp_path / "short.gguf"
    short.write_bytes(data[:len(data) - 4096])
    with pytest.raises(ValueError, match="extends past the end"):
        GGUFLoader(str(short)).load()
    assert QUANT_INFO[8] == (34, 32) and QUANT_INFO[6] == (22, 32) and QUANT_INFO[12] == (144, 256)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "adam", "loaders")), reason="no checkout of the reference")
def test_live_reference_loader_reads_the_same(golden_dir):
    sys.path.insert(0, REFERENCE)
    try:
        from adam.loaders.gguf import GGUFLoader as RefLoader
    finally:
        sys.path.remove(REFERENCE)
    path = os.path.join(golden_dir, "tiny.gguf")
    ref = RefLoader(path, keep_tensors=False, keep_raw_blocks=False)
    ref.load(verbose=False)
    ld = GGUFLoader(path).load()
    assert ref.metadata == ld.metadata and ref._data_offset == ld._data_offset
    assert {n: tuple(s) for n, s in ref.tensor_shapes.items()} == {n: tuple(s) for n, s in ld.tensor_shapes.items()}
    assert ref.tensor_types == ld.tensor_types
    for ti in ref.tensor_infos:
        assert ref.load_tensor_raw(ti.name) == ld.load_tensor_raw(ti.name).tobytes()
    ld.close()
