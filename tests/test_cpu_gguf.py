"""The GGUF reader of the C ABI against files written by gguf-py (no GPU): records, metadata, conversion to f32, shards,
and the errors of damaged files."""
import numpy as np
import pytest

from gguf_files import ARCH, model_meta, write_gguf


def _rand_blocks(rng, n, bytes_per):
    b = rng.integers(0, 256, size=(n, bytes_per), dtype=np.uint8)
    d = b[:, :2].view(np.uint16)
    d[(d & 0x7C00) == 0x7C00] &= 0x3FFF   # no inf / nan scales
    return b


@pytest.fixture(scope="module")
def sample(tmp_path_factory):
    from gguf import GGMLQuantizationType as QT
    rng = np.random.default_rng(11)
    t = {
        "a.f32": rng.standard_normal((6, 64)).astype(np.float32),
        "b.f16": rng.standard_normal((5, 32)).astype(np.float16),
        "c.q8_0": (_rand_blocks(rng, 4 * 2, 34).reshape(4, 2 * 34), QT.Q8_0),
        "d.iq3_s": (_rand_blocks(rng, 3 * 7 * 2, 110).reshape(3, 7, 2 * 110), QT.IQ3_S),
        "e.i32": np.arange(48, dtype=np.int32),
        "f.bf16": ((rng.standard_normal((3, 16)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16).view(np.uint8).reshape(3, 32), QT.BF16),
    }
    meta = {"general.name": "sample", ".block_count": 7, ".rope.freq_base": 1e7, "some.flags": [3, 1, 4, 1, 5], "some.bool": True}
    p = tmp_path_factory.mktemp("gguf") / "sample.gguf"
    write_gguf(p, meta, t)
    return p, t


def test_records_and_metadata(F, sample):
    path, t = sample
    g = F.Gguf(path)
    assert len(g) == len(t) and g.shards() == 1
    assert g.str("general.architecture") == ARCH and g.str("general.name") == "sample"
    assert g.num(ARCH + ".block_count") == 7 and g.num(ARCH + ".rope.freq_base") == pytest.approx(1e7)
    assert g.num("some.bool") == 1 and g.int_array("some.flags") == [3, 1, 4, 1, 5]
    assert g.num("no.such.key") is None and g.str("no.such.key") is None and g.find("no.such.tensor") is None
    names = sorted(g.tensor_at(i).name.decode() for i in range(len(g)))
    assert names == sorted(t)
    a = g.find("a.f32")
    assert (a.type, a.n_dims, list(a.ne)) == (0, 2, [64, 6, 1, 1]) and a.bytes == 6 * 64 * 4 and a.offset % 32 == 0
    d = g.find("d.iq3_s")
    assert (d.type, d.n_dims, list(d.ne)) == (21, 3, [512, 7, 3, 1]) and d.bytes == 3 * 7 * 2 * 110
    assert g.raw(d) == t["d.iq3_s"][0].tobytes()
    e = g.find("e.i32")
    assert e.type == 26 and np.array_equal(np.frombuffer(g.raw(e), np.int32), t["e.i32"])
    g.close()


def test_rows_to_f32_match_gguf_py(F, sample):
    from gguf import GGMLQuantizationType as QT
    from gguf.quants import dequantize
    path, t = sample
    g = F.Gguf(path)
    assert np.array_equal(g.rows_f32(g.find("a.f32")), t["a.f32"])
    assert np.array_equal(g.rows_f32(g.find("b.f16")), t["b.f16"].astype(np.float32))
    assert np.array_equal(g.rows_f32(g.find("b.f16"), 2, 2), t["b.f16"][2:4].astype(np.float32))
    q8 = dequantize(t["c.q8_0"][0], QT.Q8_0)
    assert np.array_equal(g.rows_f32(g.find("c.q8_0")).view(np.uint32), q8.view(np.uint32))
    iq = dequantize(t["d.iq3_s"][0], QT.IQ3_S).reshape(21, 512)
    assert np.array_equal(g.rows_f32(g.find("d.iq3_s")).view(np.uint32), iq.view(np.uint32))
    assert np.array_equal(g.rows_f32(g.find("d.iq3_s"), 8, 5).view(np.uint32), iq[8:13].view(np.uint32))
    bf = (t["f.bf16"][0].view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(3, 16)
    assert np.array_equal(g.rows_f32(g.find("f.bf16")).view(np.uint32), bf.view(np.uint32))
    with pytest.raises(F.FnxError, match="rows"):
        g.rows_f32(g.find("a.f32"), 4, 3)
    with pytest.raises(F.FnxError, match="type 26"):
        g.rows_f32(g.find("e.i32"))
    g.close()


def test_model_config_from_metadata(F, tmp_path):
    cfg = F.flash_next_config(n_layer=4, hidden=512, n_expert=8, top_k=2, ffn=256, n_q_head=2, n_kv_head=1, head_dim=128, n_rot=32, gdn_k_head=2,
                              gdn_v_head=4, gdn_head_dim=128, vocab=640, draft_vocab=64)
    t = {"token_embd.weight": np.zeros((cfg.vocab, cfg.hidden), np.float16), f"blk.{cfg.n_layer}.nextn.draft_vocab": np.arange(64, dtype=np.int32)}
    write_gguf(tmp_path / "m.gguf", model_meta(cfg), t)
    g = F.Gguf(tmp_path / "m.gguf")
    got = g.model_config(max_ctx=777, max_rows=6, n_seq=3)
    for name, _ in cfg._fields_:
        want = {"max_ctx": 777, "max_rows": 6, "n_seq": 3}.get(name, getattr(cfg, name))
        assert getattr(got, name) == pytest.approx(want), name
    g.close()
    meta = model_meta(cfg)
    del meta[".expert_count"]
    write_gguf(tmp_path / "m2.gguf", meta, t)
    g = F.Gguf(tmp_path / "m2.gguf")
    with pytest.raises(F.FnxError, match="expert_count"):
        g.model_config()
    g.close()


def test_shards_are_found_beside_the_first(F, tmp_path):
    a = {"x": np.arange(12, dtype=np.float32).reshape(3, 4)}
    b = {"y": np.arange(8, dtype=np.float32).reshape(2, 4) + 100}
    write_gguf(tmp_path / "m-00001-of-00002.gguf", {"general.name": "first"}, a)
    write_gguf(tmp_path / "m-00002-of-00002.gguf", {"general.name": "second"}, b)
    g = F.Gguf(tmp_path / "m-00001-of-00002.gguf")
    assert g.shards() == 2 and len(g) == 2 and g.str("general.name") == "first"
    assert g.find("x").shard == 0 and g.find("y").shard == 1
    assert np.array_equal(g.rows_f32(g.find("y")), b["y"])
    g.close()
    (tmp_path / "m-00002-of-00002.gguf").unlink()
    with pytest.raises(F.FnxError, match="cannot open"):
        F.Gguf(tmp_path / "m-00001-of-00002.gguf")


def test_damaged_files_are_refused(F, sample, tmp_path):
    path, _ = sample
    raw = path.read_bytes()
    for name, data, msg in [
        ("magic", b"GGUX" + raw[4:], "does not start with GGUF"),
        ("version", raw[:4] + (9).to_bytes(4, "little") + raw[8:], "version 9"),
        ("short", raw[:16], "too short"),
        ("meta", raw[:60], "ends inside"),
        ("data", raw[:len(raw) - 700], "past the end"),
    ]:
        p = tmp_path / (name + ".gguf")
        p.write_bytes(data)
        with pytest.raises(F.FnxError, match=msg):
            F.Gguf(p)
    with pytest.raises(F.FnxError, match="cannot open"):
        F.Gguf(tmp_path / "absent.gguf")


def _hand_written_gguf(version: int, align: int, tensors: dict, extra_meta=()):
    """A container written field by field from the format's description (no writer library): header, metadata with
    `general.alignment`, tensor records with offsets rounded up to the alignment, padded data."""
    import struct

    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    kv = [s("general.architecture") + struct.pack("<I", 8) + s("qwen3next"), s("general.alignment") + struct.pack("<II", 4, align)]
    kv += list(extra_meta)
    recs, blobs, off = [], [], 0
    for name, arr in tensors.items():
        ty = {np.dtype(np.float32): 0, np.dtype(np.float16): 1}[arr.dtype]
        recs.append(s(name) + struct.pack("<I", arr.ndim) + b"".join(struct.pack("<Q", d) for d in reversed(arr.shape)) + struct.pack("<IQ", ty, off))
        raw = arr.tobytes()
        raw += b"\0" * (-len(raw) % align)
        blobs.append(raw)
        off += len(raw)
    head = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(kv)) + b"".join(kv) + b"".join(recs)
    head += b"\0" * (-len(head) % align)
    return head + b"".join(blobs)


@pytest.mark.parametrize("version,align", [(3, 32), (3, 64), (2, 32), (3, 4096)])
def test_alignment_key_and_version_2(F, tmp_path, version, align):
    import struct
    rng = np.random.default_rng(align + version)
    tensors = {"a": rng.standard_normal((3, 5)).astype(np.float32), "b": rng.standard_normal((7, 2)).astype(np.float16),
               "c": rng.standard_normal((1, 33)).astype(np.float32)}
    name = "general.name".encode()
    extra = [struct.pack("<Q", len(name)) + name + struct.pack("<I", 8) + struct.pack("<Q", 4) + b"hand"]
    p = tmp_path / "hand.gguf"
    p.write_bytes(_hand_written_gguf(version, align, tensors, extra))
    g = F.Gguf(p)
    assert len(g) == 3 and g.str("general.name") == "hand" and g.num("general.alignment") == align
    for k, want in tensors.items():
        t = g.find(k)
        assert t is not None and t.n_dims == want.ndim and tuple(t.ne[: want.ndim]) == tuple(reversed(want.shape))
        assert np.array_equal(g.rows_f32(t), want.astype(np.float32))
    g.close()
