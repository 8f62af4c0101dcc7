"""GGUF container and block codecs (CPU)."""
import numpy as np
import pytest
import torch

from openagents_b200.gguf import GGUFFile, GGUFWriter, GgmlType, dequantize, quantize, tensor_nbytes
from openagents_b200.gguf import torch_codecs as tc

BLOCK_BYTES = {GgmlType.Q8_0: (32, 34), GgmlType.Q4_K: (256, 144), GgmlType.Q5_K: (256, 176),
               GgmlType.Q6_K: (256, 210), GgmlType.MXFP4: (32, 17)}
# RMS error relative to the data's std, generous upper bounds per format
ERR_BOUND = {GgmlType.F32: 0, GgmlType.F16: 1e-3, GgmlType.BF16: 4e-3, GgmlType.Q8_0: 1e-2, GgmlType.Q6_K: 3e-2,
             GgmlType.Q5_K: 6e-2, GgmlType.Q4_K: 1.2e-1, GgmlType.MXFP4: 2e-1}


def _x(shape=(16, 1024), seed=0):
    return (np.random.default_rng(seed).standard_normal(shape) * 0.02).astype(np.float32)


@pytest.mark.parametrize("t", list(GgmlType))
def test_quant_roundtrip_error(t):
    x = _x()
    q = quantize(x, t)
    assert q.size == tensor_nbytes(t, x.size)
    y = dequantize(q, t, x.shape)
    rel = float(np.sqrt(((x - y) ** 2).mean()) / x.std())
    assert rel <= ERR_BOUND[t] + 1e-12
    # quantizing the dequantized values again is a fixed point for the scalar formats
    if t in (GgmlType.F16, GgmlType.BF16, GgmlType.Q8_0):
        assert np.array_equal(dequantize(quantize(y, t), t, x.shape), y)


@pytest.mark.parametrize("t,bb", list(BLOCK_BYTES.items()))
def test_block_sizes(t, bb):
    assert tensor_nbytes(t, bb[0] * 3) == bb[1] * 3
    with pytest.raises(ValueError):
        tensor_nbytes(t, bb[0] + 1)


def test_q4k_known_block():
    """Hand-built superblock: d=1, dmin=0.5, scale j -> j+1, min j -> j, nibble l -> l % 16."""
    blk = np.zeros(144, dtype=np.uint8)
    blk[0:2] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
    blk[2:4] = np.frombuffer(np.float16(0.5).tobytes(), dtype=np.uint8)
    ls, lm = [j + 1 for j in range(8)], list(range(8))
    sc = blk[4:16]
    for j in range(8):
        if j < 4:
            sc[j] |= ls[j]
            sc[j + 4] |= lm[j]
        else:
            sc[j + 4] = (ls[j] & 0xF) | ((lm[j] & 0xF) << 4)
            sc[j - 4] |= (ls[j] >> 4) << 6
            sc[j] |= (lm[j] >> 4) << 6
    for g in range(4):
        for l in range(32):
            blk[16 + 32 * g + l] = (l % 16) | (((l + 3) % 16) << 4)
    y = dequantize(blk, GgmlType.Q4_K, (256,))
    for g in range(4):
        for l in range(32):
            assert y[64 * g + l] == ls[2 * g] * (l % 16) - 0.5 * lm[2 * g]
            assert y[64 * g + 32 + l] == ls[2 * g + 1] * ((l + 3) % 16) - 0.5 * lm[2 * g + 1]


def test_mxfp4_values():
    blk = np.zeros(17, dtype=np.uint8)
    blk[0] = 128  # 2^1
    for j in range(16):
        blk[1 + j] = j | ((15 - j) << 4)
    y = dequantize(blk, GgmlType.MXFP4, (32,))
    lut = [0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6]
    assert [float(v) for v in y[:16]] == [2 * lut[j] for j in range(16)]
    assert [float(v) for v in y[16:]] == [2 * lut[15 - j] for j in range(16)]


def test_file_roundtrip(tmp_path):
    p = str(tmp_path / "m.gguf")
    x = _x((8, 512))
    w = GGUFWriter(p)
    w.add_meta("general.architecture", "llama")
    w.add_meta("llama.block_count", 2)
    w.add_meta("llama.rope.freq_base", 500000.0)
    w.add_meta("tokenizer.ggml.tokens", ["<s>", "a\"b", "日本"])
    w.add_meta("some.ints", [1, -2, 3])
    w.add_meta("flag", True)
    packed = {}
    for t in (GgmlType.F32, GgmlType.F16, GgmlType.BF16, GgmlType.Q8_0, GgmlType.Q4_K, GgmlType.Q6_K, GgmlType.MXFP4):
        packed[t] = quantize(x, t)
        w.add_tensor_raw(f"t.{t.name}", t, x.shape, packed[t])
    w.write()
    with GGUFFile(p) as f:
        assert f.version == 3 and f.architecture == "llama"
        assert f.metadata["llama.block_count"] == 2 and f.metadata["flag"] is True
        assert f.metadata["tokenizer.ggml.tokens"] == ["<s>", "a\"b", "日本"]
        assert f.metadata["some.ints"] == [1, -2, 3]
        for t, b in packed.items():
            ten = f.tensors[f"t.{t.name}"]
            assert ten.shape == x.shape and ten.type == t
            assert ten.offset % f.alignment == 0
            assert np.array_equal(ten.data, b)          # save -> load is bitwise
    # re-save what was loaded: identical bytes on disk
    p2 = str(tmp_path / "m2.gguf")
    with GGUFFile(p) as f:
        w = GGUFWriter(p2)
        for k, v in f.metadata.items():
            w.add_meta(k, v, kind="f32" if isinstance(v, float) else None)
        for n, ten in f.tensors.items():
            w.add_tensor_raw(n, ten.type, ten.shape, ten.data.copy())
        w.write()
    assert open(p, "rb").read() == open(p2, "rb").read()


def test_bad_files(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"NOPE" + b"\0" * 64)
    with pytest.raises(ValueError):
        GGUFFile(str(p))
    p.write_bytes(b"GGUF" + (3).to_bytes(4, "little") + (1).to_bytes(8, "little") + (0).to_bytes(8, "little"))
    with pytest.raises(ValueError):
        GGUFFile(str(p))


@pytest.mark.parametrize("t", [GgmlType.Q8_0, GgmlType.Q4_K, GgmlType.Q6_K, GgmlType.MXFP4])
def test_torch_codecs_match_cpp(t):
    x = torch.from_numpy(_x((32, 1024), seed=3))
    a = torch.from_numpy(quantize(x.numpy(), t))
    b = tc.quantize(x, t)
    assert torch.equal(a, b)
    assert torch.equal(tc.dequantize(b, t, x.shape), torch.from_numpy(dequantize(b.numpy(), t, x.shape)))


def test_repack_roundtrip_and_orders():
    x = torch.from_numpy(_x((4, 512), seed=5))
    b = tc.quantize(x, GgmlType.Q4_K)
    r = tc.repack_q4_k(b)
    assert r.numel() == b.numel() and torch.equal(tc.unpack_q4_k_r(r), b)
    # the pair extraction the tensor-core dequant uses yields elements in order
    w = r.reshape(-1, 144)[:, 16:].contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    pairs = [((w >> (4 * s)) & 0x000F000F) for s in range(4)]
    el = torch.stack([v for p in pairs for v in (p & 0xF, p >> 16)], -1).reshape(-1, 256)
    qs = b.reshape(-1, 144)[:, 16:].reshape(-1, 4, 32)
    L = torch.stack((qs & 0xF, qs >> 4), 2).reshape(-1, 256).long()
    assert torch.equal(el, L)
    assert tc.X8_POS == (0, 2, 4, 6, 1, 3, 5, 7)


def test_corrupt_headers_are_errors_not_crashes(tmp_path):
    """Header counts and tensor extents are checked against the file size with overflow-safe arithmetic."""
    import struct
    from openagents_b200.gguf import GGUFFile

    def write(name, body):
        p = tmp_path / name
        p.write_bytes(b"GGUF" + struct.pack("<I", 3) + body)
        return str(p)

    # counts far beyond what the file could hold
    with pytest.raises(Exception, match="counts exceed|malformed|truncated"):
        GGUFFile(write("huge_counts.gguf", struct.pack("<QQ", 2 ** 60, 0) + b"\0" * 64))
    with pytest.raises(Exception, match="counts exceed|malformed|truncated"):
        GGUFFile(write("huge_kv.gguf", struct.pack("<QQ", 0, 2 ** 61) + b"\0" * 64))
    # one tensor whose dimensions multiply past 64 bits
    name = b"t"
    info = struct.pack("<Q", len(name)) + name + struct.pack("<I", 2) + struct.pack("<QQ", 2 ** 40, 2 ** 40) + struct.pack("<IQ", 0, 0)
    with pytest.raises(Exception, match="impossible element count|past the end"):
        GGUFFile(write("overflow_dims.gguf", struct.pack("<QQ", 1, 0) + info + b"\0" * 64))
    # an offset chosen so that offset + size wraps around
    info = struct.pack("<Q", len(name)) + name + struct.pack("<I", 1) + struct.pack("<Q", 32) + struct.pack("<IQ", 0, 2 ** 64 - 64)
    with pytest.raises(Exception, match="past the end"):
        GGUFFile(write("wrap_offset.gguf", struct.pack("<QQ", 1, 0) + info + b"\0" * 256))


def test_command_line_inspect_quantize_digest(tmp_path, capsys):
    import json
    from openagents_b200.gguf.__main__ import main
    from openagents_b200.models.config import TINY_LLAMA
    from openagents_b200.models.weights import PLAN_BF16, load_gguf_float, random_weights, save_gguf
    cfg = TINY_LLAMA.with_(vocab=512, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512)
    src, dst = str(tmp_path / "a.gguf"), str(tmp_path / "b.gguf")
    save_gguf(src, cfg, random_weights(cfg, 0), PLAN_BF16, extra_meta={"tokenizer.b200.byte_bpe": '{"schema": "x"}', "general.author": "someone"})
    assert main(["inspect", src]) == 0
    a = json.loads(capsys.readouterr().out)
    assert a["architecture"] == "llama" and a["tokenizer"] == "b200-byte-bpe" and list(a["byType"]) == ["BF16"] or "F32" in a["byType"]
    assert a["bitsPerWeight"] >= 16.0 and a["shape"]["block_count"] == cfg.n_layers
    assert main(["quantize", src, dst, "--plan", "q4_k"]) == 0
    q = json.loads(capsys.readouterr().out)
    assert 0.0 < q["worstRelativeRmsError"] < 0.12 and q["tensorBytes"] < a["tensorBytes"] / 2.5
    assert "tokenizer.b200.byte_bpe" in q["keptMetadataKeys"] and "general.author" in q["keptMetadataKeys"]
    assert {r["to"] for r in q["tensors"]} >= {"Q4_K", "Q6_K"}
    main(["inspect", dst])
    b = json.loads(capsys.readouterr().out)
    assert b["bitsPerWeight"] < 7.0 and b["tokenizer"] == "b200-byte-bpe" and b["shape"] == a["shape"]
    c2, w2 = load_gguf_float(dst)
    assert c2.d_model == 256 and set(w2) == set(random_weights(cfg, 0))
    main(["digest", dst])
    assert json.loads(capsys.readouterr().out)["artifactDigest"].startswith("sha256:")
