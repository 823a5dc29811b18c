"""The on-disk side of the frozen-linear path (caif_b200/host/caif_safetensors.hpp): SafeTensors files with the
reference's dtype vocabulary (I8, and I4 at two codes per byte), checkpoint directories, the Hugging Face <-> CAIF
name mapper, and loading a frozen linear straight from a file.

Checked against three things: the `safetensors` Python package (standard dtypes, both directions), the
reference's own reader / writer / mapper (oracle/_ref/libcaif_ref_layers.so: header parsing and the mapper run
without a device, Save / Load on the GPU), and golden files the reference produced
(tests/golden/weight_mapper.json, tests/golden/reference_written.safetensors; tests/golden/make_format_golden.py)."""
import json
import os
import struct
import sys

import numpy as np
import pytest
import torch

import caif_oracle as orc
import reflayers as rl
from caif_b200 import host_layers as hl
from caif_b200 import native as nv

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)
import make_format_golden as mfg  # noqa: E402


def _write_raw(path, header_text, payload=b"", header_len=None):
    raw = header_text.encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw) if header_len is None else header_len))
        f.write(raw)
        f.write(payload)


def _mine(cases):
    return [(name, mfg.NAMES[code], shape, data) for name, code, shape, data in cases]


def test_written_file_layout_and_round_trip(tmp_path):
    path = str(tmp_path / "a.safetensors")
    cases = mfg.format_cases() + [("empty", mfg.I8, [0, 4], b"")]
    hl.save_safetensors(path, _mine(cases), mfg.METADATA)
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    assert hlen % 8 == 0 and raw[8 + hlen - 1:8 + hlen] in (b" ", b"}")
    header = json.loads(raw[8:8 + hlen])
    assert list(header)[-1] == "__metadata__" and header["__metadata__"] == mfg.METADATA
    cursor = 0
    for name, code, shape, data in cases:            # back to back, in the order given
        assert header[name] == {"dtype": mfg.NAMES[code], "shape": shape, "data_offsets": [cursor, cursor + len(data)]}
        assert raw[8 + hlen + cursor:8 + hlen + cursor + len(data)] == data
        cursor += len(data)
    assert len(raw) == 8 + hlen + cursor
    f = hl.SafeTensors(path)
    assert f.names() == [c[0] for c in cases]
    assert f.metadata() == mfg.METADATA
    for name, code, shape, data in cases:
        info = f.info(name)
        assert (info["dtype"], info["shape"], info["bytes"]) == (mfg.NAMES[code], shape, len(data))
        assert f.read(name) == data
    assert f.info("q.int4")["bytes"] == 8              # 15 codes: (15 + 1) / 2
    with pytest.raises(hl.HostLayerError, match="not found"):
        f.info("absent")
    f.close()


def test_interoperates_with_the_safetensors_package(tmp_path):
    from safetensors import safe_open
    from safetensors.numpy import save_file
    from safetensors.torch import load_file

    cases = [c for c in mfg.format_cases() if c[1] != mfg.I4]     # the package has no I4
    mine = str(tmp_path / "mine.safetensors")
    hl.save_safetensors(mine, _mine(cases), {"framework": "CAIF"})
    loaded = load_file(mine)
    views = {mfg.F32: torch.float32, mfg.F16: torch.float16, mfg.BF16: torch.bfloat16, mfg.I8: torch.int8}
    for name, code, shape, data in cases:
        assert loaded[name].dtype == views[code] and list(loaded[name].shape) == shape
        assert loaded[name].contiguous().view(torch.uint8).numpy().tobytes() == data
    with safe_open(mine, framework="numpy") as g:
        assert g.metadata() == {"framework": "CAIF"}
    theirs = str(tmp_path / "theirs.safetensors")
    arrays = {"b.w": np.arange(12, dtype=np.float32).reshape(3, 4), "a.q": np.arange(-5, 5, dtype=np.int8),
              "c.h": np.linspace(0, 1, 6, dtype=np.float16).reshape(2, 3), "d.i": np.arange(4, dtype=np.int64)}
    save_file(arrays, theirs, metadata={"format": "pt", "unicode": "café ☃"})
    f = hl.SafeTensors(theirs)
    assert sorted(f.names()) == sorted(arrays)
    assert f.metadata() == {"format": "pt", "unicode": "café ☃"}
    for name, arr in arrays.items():
        assert f.read(name) == arr.tobytes() and f.info(name)["shape"] == list(arr.shape)
    assert f.info("d.i")["dtype"] == "I64"             # readable as bytes although no device tensor type exists
    f.close()


def test_header_parsing_equals_the_reference(tmp_path):
    if not rl.available():
        pytest.skip("reference library not built")
    path = str(tmp_path / "a.safetensors")
    hl.save_safetensors(path, _mine(mfg.format_cases()), mfg.METADATA)
    f = hl.SafeTensors(path)
    want = rl.st_tensor_infos(path)
    assert sorted(want) == sorted(f.names())
    for name, (dtype, shape, begin, end) in want.items():
        info = f.info(name)
        assert (info["dtype"], info["shape"], info["begin"], info["end"]) == (dtype, shape, begin, end)
    assert rl.st_metadata(path) == f.metadata()
    f.close()


def test_golden_file_written_by_the_reference():
    path = os.path.join(GOLDEN, "reference_written.safetensors")
    if not os.path.exists(path):
        pytest.skip("golden file not generated yet")
    f = hl.SafeTensors(path)
    cases = mfg.format_cases()
    assert f.names() == [c[0] for c in cases]
    assert f.metadata() == mfg.METADATA
    for name, code, shape, data in cases:
        assert f.read(name) == data and f.info(name)["dtype"] == mfg.NAMES[code] and f.info(name)["shape"] == shape
    f.close()


def test_writer_reproduces_the_reference_file_byte_for_byte(tmp_path):
    path = os.path.join(GOLDEN, "reference_written.safetensors")
    if not os.path.exists(path):
        pytest.skip("golden file not generated yet")
    mine = str(tmp_path / "mine.safetensors")
    hl.save_safetensors(mine, _mine(mfg.format_cases()), mfg.METADATA)
    assert open(mine, "rb").read() == open(path, "rb").read()


@pytest.mark.parametrize("case,match", [
    ("tiny", "file too small"),
    ("huge_header", "header too large"),
    ("header_past_end", "invalid header size"),
    ("bad_json", "malformed JSON"),
    ("size_mismatch", "data size mismatch"),
    ("reversed", "data_offset_start exceeds data_offset_end"),
    ("past_end", "extends past end of file"),
    ("unknown_dtype", "unrecognised name"),
])
def test_malformed_files_are_refused(tmp_path, case, match):
    """The refusals of src/caif_safetensors_format.cpp:262-359, same messages."""
    path = str(tmp_path / "bad.safetensors")
    entry = '{"t":{"dtype":"%s","shape":[2,2],"data_offsets":[%d,%d]}}'
    if case == "tiny":
        open(path, "wb").write(b"\x01\x02\x03")
    elif case == "huge_header":
        _write_raw(path, "{}", header_len=200 * 1024 * 1024)
    elif case == "header_past_end":
        _write_raw(path, "{}", header_len=64)
    elif case == "bad_json":
        _write_raw(path, '{"t":{"dtype":"F32","shape":[2,2]')
    elif case == "size_mismatch":
        _write_raw(path, entry % ("F32", 0, 12), b"\0" * 16)
    elif case == "reversed":
        _write_raw(path, entry % ("F32", 16, 0), b"\0" * 16)
    elif case == "past_end":
        _write_raw(path, entry % ("F32", 0, 16), b"\0" * 8)
    elif case == "unknown_dtype":
        _write_raw(path, entry % ("Q7", 0, 16), b"\0" * 16)
    with pytest.raises(hl.HostLayerError, match=match):
        f = hl.SafeTensors(path)
        f.read("t")
    if rl.available() and case in ("tiny", "huge_header", "header_past_end"):
        with pytest.raises(RuntimeError):     # the reference refuses the same files (its exception type carries
            rl.st_tensor_infos(path)          # the same text but is not a std::exception the doorway can read)


def test_too_many_tensors_is_refused(tmp_path):
    with pytest.raises(hl.HostLayerError, match="too many tensors"):
        hl.save_safetensors(str(tmp_path / "many.safetensors"), [("t%d" % i, "I8", [1], b"\0") for i in range(4097)])


def test_checkpoint_directory_with_index_and_single_file(tmp_path):
    cases = _mine(mfg.format_cases())
    sharded = tmp_path / "sharded"
    sharded.mkdir()
    hl.save_safetensors(str(sharded / "model-00001-of-00002.safetensors"), cases[:3])
    hl.save_safetensors(str(sharded / "model-00002-of-00002.safetensors"), cases[3:])
    weight_map = {c[0]: "model-00001-of-00002.safetensors" for c in cases[:3]}
    weight_map.update({c[0]: "model-00002-of-00002.safetensors" for c in cases[3:]})
    (sharded / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": 1},
                                                                      "weight_map": weight_map}, indent=2))
    d = hl.SafeTensors(str(sharded), directory=True)
    assert d.names() == sorted(weight_map)
    for name, dtype, shape, data in cases:
        assert d.read(name) == data
        assert os.path.basename(d.info(name)["file"]) == weight_map[name]
    with pytest.raises(hl.HostLayerError, match="not found in weight map"):
        d.read("absent")
    d.close()
    single = tmp_path / "single"
    single.mkdir()
    hl.save_safetensors(str(single / "model.safetensors"), cases)
    d = hl.SafeTensors(str(single), directory=True)
    assert d.read("q.int4") == cases[4][3]
    d.close()
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(hl.HostLayerError, match="no index file and no model.safetensors"):
        hl.SafeTensors(str(empty), directory=True)
    (empty / "model.safetensors.index.json").write_text('{"weight_map": {}}')
    with pytest.raises(hl.HostLayerError, match="empty weight map"):
        hl.SafeTensors(str(empty), directory=True)


def _mapper_answers():
    m = hl.WeightMapper()

    def add(alias, hf, aif):
        (m.add_alias if alias else m.add_prefix_rule)(hf, aif)

    def translate(hf_to_aif, name):
        return m.hf_to_aif(name) if hf_to_aif else m.aif_to_hf(name)

    answers = mfg.mapper_answers(add, translate, m._query)
    m.close()
    return answers


def test_weight_mapper_against_the_golden_answers_of_the_reference():
    want = json.load(open(os.path.join(GOLDEN, "weight_mapper.json")))
    assert _mapper_answers() == want


def test_weight_mapper_against_the_reference_on_random_rules():
    if not rl.available():
        pytest.skip("reference library not built")
    rng = np.random.default_rng(8)
    parts = ["model", "layers", "mlp", "attn", "0", "1", "12", "weight", "up", "down", "x"]

    def name(n):
        return ".".join(rng.choice(parts, n)) + ("." if rng.random() < 0.5 else "")

    mine, theirs = hl.WeightMapper(), rl.Mapper()
    seen_hf, seen_aif = set(), set()
    for _ in range(12):
        hf, aif = name(int(rng.integers(1, 4))), name(int(rng.integers(1, 4)))
        # two rules with one prefix of equal length have no defined winner in either implementation
        if hf in seen_hf or aif in seen_aif:
            continue
        seen_hf.add(hf)
        seen_aif.add(aif)
        alias = bool(rng.random() < 0.3)
        (mine.add_alias if alias else mine.add_prefix_rule)(hf, aif)
        theirs.add(alias, hf, aif)
    probes = [name(int(rng.integers(1, 6))) + "tail" for _ in range(300)] + sorted(seen_hf) + sorted(seen_aif)
    for p in probes:
        assert mine.hf_to_aif(p) == theirs.translate(1, p)
        assert mine.aif_to_hf(p) == theirs.translate(0, p)
    assert mine.missing_names(probes[:50], probes[50:100]) == theirs.query(0, probes[:50], probes[50:100])
    assert mine.unmapped_hf_names(probes) == theirs.query(1, [], probes)
    mine.close()
    theirs.close()


# ------------------------------------------------------------------------------------------ on the GPU
@pytest.mark.gpu
def test_files_cross_between_this_library_and_the_reference(tmp_path):
    """The reference's Save -> this reader, and this library's device Save -> the reference's Load: same bytes,
    including the odd-length I4 tensor; the two writers produce byte-identical files."""
    if not rl.available():
        pytest.skip("reference library not built")
    cases = mfg.format_cases()
    theirs = str(tmp_path / "theirs.safetensors")
    rl.st_save(theirs, cases, mfg.METADATA)
    f = hl.SafeTensors(theirs)
    assert f.names() == [c[0] for c in cases] and f.metadata() == mfg.METADATA
    for name, code, shape, data in cases:
        assert f.read(name) == data
        assert f.load_device(name).cpu().numpy().tobytes() == data
    f.close()
    mine_host = str(tmp_path / "mine_host.safetensors")
    hl.save_safetensors(mine_host, _mine(cases), mfg.METADATA)
    assert open(mine_host, "rb").read() == open(theirs, "rb").read()
    mine = str(tmp_path / "mine.safetensors")
    held = [torch.frombuffer(bytearray(c[3]), dtype=torch.uint8).cuda() for c in cases]
    hl.save_safetensors_device(mine, [(c[0], c[1], c[2], t) for c, t in zip(cases, held)])
    for name, code, shape, data in cases:
        got_code, got = rl.st_load(mine, name, 4096)
        assert got_code == code and got == data
    single = tmp_path / "dir"
    single.mkdir()
    hl.save_safetensors(str(single / "model.safetensors"), _mine(cases))
    assert rl.st_load(str(single), "q.int4", 4096, from_directory=True)[1] == cases[4][3]


@pytest.mark.gpu
@pytest.mark.parametrize("storage", [orc.I4, orc.I8, orc.BF16, orc.F32])
def test_frozen_linear_loaded_from_a_file(tmp_path, storage):
    """LoadFrozenLinear: codes + scales as stored give the layer the ordinary loading path gives (bit-equal
    outputs); a float weight in the file is quantized (or converted) on the device at load time and gives what
    quantizing first and loading the codes gives."""
    from gpu_util import act, make_weight

    rng = np.random.default_rng(11 + storage)
    in_dim, out_dim, m = 256, 96, 40
    weight, codes, scales = make_weight(rng, out_dim, in_dim, storage)
    st_name = {orc.I4: "I4", orc.I8: "I8", orc.BF16: "BF16", orc.F32: "F32"}[storage]
    w_f32 = (rng.standard_normal((out_dim, in_dim)) * 0.05).astype(np.float32)
    tensors = [("blk.w", st_name, [in_dim, out_dim], weight.codes.contiguous().view(torch.uint8).cpu().numpy().tobytes()),
               ("blk.w_f32", "F32", [in_dim, out_dim], w_f32.tobytes()),
               ("blk.w_bf16", "BF16", [in_dim, out_dim],
                torch.from_numpy(w_f32).to(torch.bfloat16).view(torch.int16).numpy().tobytes())]
    if scales is not None:
        sc = np.ascontiguousarray(scales)
        tensors.append(("blk.w.scales", "F16" if storage == orc.I4 else "F32", [sc.size], sc.tobytes()))
    path = str(tmp_path / "layer.safetensors")
    hl.save_safetensors(path, tensors)
    f = hl.SafeTensors(path)
    _, x = act(rng, m, in_dim, orc.BF16)

    plain = hl.Layer(in_dim, out_dim, storage, compute=nv.BF16)
    plain.load_weight(weight.codes, storage)
    if scales is not None:
        plain.load_scales_from_host(np.ascontiguousarray(scales).tobytes())
    from_file = hl.Layer(in_dim, out_dim, storage, compute=nv.BF16)
    if scales is not None:
        with pytest.raises(hl.HostLayerError, match="needs a scales tensor"):
            f.load_frozen_linear(from_file, "blk.w")
    f.load_frozen_linear(from_file, "blk.w", "blk.w.scales" if scales is not None else "")
    assert torch.equal(from_file.forward(x), plain.forward(x))

    # a float tensor in the file, this layer's storage
    for src in ("blk.w_f32", "blk.w_bf16"):
        src_f32 = torch.from_numpy(w_f32).cuda() if src == "blk.w_f32" else \
            torch.from_numpy(w_f32).to(torch.bfloat16).float().cuda()
        direct = hl.Layer(in_dim, out_dim, storage, compute=nv.BF16)
        if storage == orc.I4:
            pk, sc = nv.quantize_int4(src_f32.reshape(-1), 128)
            direct.load_weight(pk, nv.I4)
            direct.load_scales_from_host(sc.cpu().numpy().tobytes())
        elif storage == orc.I8:
            q, sc = nv.quantize_int8_per_tensor(src_f32.reshape(-1))
            direct.load_weight(q, nv.I8)
            direct.load_scales_from_host(sc.cpu().numpy().tobytes())
        else:
            direct.load_weight(src_f32.to(nv._CODE_TO_TORCH[storage]).contiguous(), storage)
        loaded = hl.Layer(in_dim, out_dim, storage, compute=nv.BF16)
        f.load_frozen_linear(loaded, src)
        assert torch.equal(loaded.forward(x), direct.forward(x))
        loaded.close()
        direct.close()
    wrong = hl.Layer(in_dim, out_dim, orc.I8 if storage != orc.I8 else orc.I4, compute=nv.BF16)
    if storage in (orc.I4, orc.I8):
        with pytest.raises(hl.HostLayerError, match="the layer stores"):
            f.load_frozen_linear(wrong, "blk.w", "blk.w.scales")
    for layer in (plain, from_file, wrong):
        layer.close()
    f.close()


def test_random_files_cross_with_the_safetensors_package(tmp_path):
    """Seeded random tensor sets (odd names with quotes, backslashes and non-ASCII characters, scalar-like and
    zero-sized shapes, every standard dtype this library moves) written by one side and read by the other."""
    from safetensors import safe_open
    from safetensors.numpy import save_file

    rng = np.random.default_rng(99)
    np_types = {"F32": np.float32, "F16": np.float16, "I8": np.int8, "U8": np.uint8, "I32": np.int32, "I64": np.int64,
                "F64": np.float64, "I16": np.int16}
    alphabet = ["w", "layer", "0", "é", "ß", "weight", "q\"uote", "back\\slash", "tab\tbed", "модель", "層"]
    for case in range(12):
        tensors, arrays = [], {}
        for t in range(int(rng.integers(1, 9))):
            name = ".".join(rng.choice(alphabet, int(rng.integers(1, 4)))) + ".%d" % t
            dtype = str(rng.choice(list(np_types)))
            shape = [int(d) for d in rng.integers(0, 5, int(rng.integers(1, 4)))]
            arr = (rng.standard_normal(shape) * 50).astype(np_types[dtype])
            arrays[name] = arr
            tensors.append((name, dtype, shape, arr.tobytes()))
        meta = {"k%d" % i: "v \" \\ %d é" % i for i in range(int(rng.integers(0, 3)))}
        mine = str(tmp_path / ("mine%d.safetensors" % case))
        hl.save_safetensors(mine, tensors, meta)
        with safe_open(mine, framework="numpy") as g:
            assert sorted(g.keys()) == sorted(arrays)
            assert (g.metadata() or {}) == meta
            for name, arr in arrays.items():
                got = g.get_tensor(name)
                assert got.dtype == arr.dtype and got.shape == arr.shape and got.tobytes() == arr.tobytes()
        theirs = str(tmp_path / ("theirs%d.safetensors" % case))
        save_file(arrays, theirs, metadata=meta or None)
        f = hl.SafeTensors(theirs)
        assert sorted(f.names()) == sorted(arrays) and f.metadata() == meta
        for name, arr in arrays.items():
            info = f.info(name)
            assert info["shape"] == list(arr.shape) and f.read(name) == arr.tobytes()
        f.close()


def test_index_file_with_escaped_names(tmp_path):
    """Hugging Face writes model.safetensors.index.json with json.dumps, which escapes non-ASCII characters as
    \\uXXXX (surrogate pairs beyond the basic plane): the names must come out as the UTF-8 strings the shard holds."""
    names = ["blöcke.0.w", "層.1.w", "emoji.\U0001F600.w"]
    d = tmp_path / "ckpt"
    d.mkdir()
    hl.save_safetensors(str(d / "shard.safetensors"), [(n, "I8", [3], bytes([i, i + 1, i + 2])) for i, n in enumerate(names)])
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {n: "shard.safetensors" for n in names}}))
    assert "\\u" in (d / "model.safetensors.index.json").read_text()
    f = hl.SafeTensors(str(d), directory=True)
    assert f.names() == sorted(names)
    for i, n in enumerate(names):
        assert f.read(n) == bytes([i, i + 1, i + 2])
    f.close()
