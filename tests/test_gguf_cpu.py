"""The native GGUF reader (`qk_gguf_*`) against files written by the test-side writer and by
gguf-py: header versions, metadata of every value type skipped correctly, alignment, tensor
registry.  No GPU needed: parsing never touches CUDA."""
import os

import numpy as np
import pytest

import gguf_writer as W
from oxillama_b200 import synth as S


def _file(tmp_path, version=3, alignment=None):
    tensors = [
        ("blk.0.ffn_up.weight", (64, 512), S.Q4_K, S.gen_weight(S.Q4_K, 64, 512, seed=1)),
        ("blk.0.ffn_down.weight", (32, 64), S.Q8_0, S.gen_weight(S.Q8_0, 32, 64, seed=2)),
        ("output_norm.weight", (32,), 0, np.zeros(32 * 4, np.uint8)),           # F32: not served here
        ("output.weight", (16, 256), S.Q6_K, S.gen_weight(S.Q6_K, 16, 256, seed=3)),
    ]
    meta = [("general.architecture", "str", "llama"), ("llama.block_count", "u32", 1),
            ("tokenizer.ggml.tokens", "arr", ("str", ["a", "bc", "def"])),
            ("tokenizer.ggml.scores", "arr", ("f32", [0.5, 1.5])), ("some.flag", "bool", 1),
            ("some.i64", "i64", -5), ("some.f64", "f64", 2.5), ("nested", "arr", ("arr", [("u8", [1, 2]), ("u8", [3])]))]
    path = os.path.join(tmp_path, f"t{version}_{alignment}.gguf")
    offs = W.write_gguf(path, tensors, meta, version=version, alignment=alignment)
    return path, tensors, offs


@pytest.mark.parametrize("version,alignment", [(3, None), (3, 64), (2, None)])
def test_tensor_registry(tmp_path, version, alignment):
    from oxillama_b200.gguf import GgufFile
    path, tensors, offs = _file(str(tmp_path), version, alignment)
    g = GgufFile(path)
    assert g.names() == [t[0] for t in tensors]
    for name, dims, type_id, data in tensors:
        info = g.info(name)
        assert (info.n_dims, info.dims, info.tensor_type) == (len(dims), tuple(dims), type_id)
        assert info.file_offset == offs[name]
        assert info.nbytes == (len(data) if type_id != 0 else 0)   # tensor_info.rs:47-56 for the served types
        with open(path, "rb") as f:
            f.seek(info.file_offset)
            assert f.read(len(data)) == np.asarray(data, np.uint8).tobytes()
    with pytest.raises(KeyError):
        g.info("no.such.tensor")
    g.close()


def test_gguf_py_file(tmp_path):
    """A file written by gguf-py (an independent writer): same registry as gguf-py's own reader sees."""
    gguf = pytest.importorskip("gguf")
    from oxillama_b200.gguf import GgufFile
    path = os.path.join(str(tmp_path), "py.gguf")
    w = gguf.GGUFWriter(path, "llama")
    w.add_block_count(2)
    w.add_token_list(["x", "yy"])
    a = S.gen_weight(S.Q4_K, 8, 256, seed=5).reshape(8, 144)
    b = S.gen_weight(S.Q8_0, 4, 64, seed=6).reshape(4, 68)
    w.add_tensor("a.weight", a, raw_dtype=gguf.GGMLQuantizationType.Q4_K)
    w.add_tensor("b.weight", b, raw_dtype=gguf.GGMLQuantizationType.Q8_0)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    r = gguf.GGUFReader(path)
    g = GgufFile(path)
    assert g.names() == [t.name for t in r.tensors]
    for t in r.tensors:
        info = g.info(t.name)
        assert info.tensor_type == int(t.tensor_type)
        assert info.file_offset == int(t.data_offset)
        assert info.nbytes == int(t.n_bytes)
        assert info.dims == tuple(int(d) for d in t.shape)
    g.close()


def test_malformed_files(tmp_path):
    from oxillama_b200.gguf import GgufFile
    from oxillama_b200.kernels import QuantError
    path, _, _ = _file(str(tmp_path))
    blob = open(path, "rb").read()
    cases = {"magic": b"GGUX" + blob[4:], "version": blob[:4] + (9).to_bytes(4, "little") + blob[8:],
             "cut_in_metadata": blob[:60], "cut_in_tensor_infos": blob[:300]}
    for name, data in cases.items():
        p = os.path.join(str(tmp_path), name + ".gguf")
        open(p, "wb").write(data)
        with pytest.raises(QuantError):
            GgufFile(p)
    with pytest.raises(QuantError):
        GgufFile(os.path.join(str(tmp_path), "missing.gguf"))
