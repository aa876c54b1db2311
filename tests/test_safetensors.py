"""Weight ingest (vAi vai/engine/safetensors-parser.cpp, weights.h, tensor.cpp:183-312,
models/production/llama3/meta-weights.h): the Python and C++ readers on synthetic
checkpoints — header parsing, the dtype conversions against the oracle's restatement of the
loader's rules, concat / slice, the Llama key map with and without a column split — and,
on the GPU, file -> device through the pinned staging ring."""
import json
import os
import struct
import subprocess

import numpy as np
import pytest

from oracle import linear_oracle as orc
from vai_b200 import Dtype
from vai_b200 import safetensors as st

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORC_DT = {Dtype.F32: orc.F32, Dtype.F16: orc.F16, Dtype.BF16: orc.BF16}


def _values(rng, shape):
    """Normal values plus the cases the conversions treat specially."""
    a = rng.standard_normal(shape).astype(np.float32)
    flat = a.reshape(-1)
    special = np.array([0.0, -0.0, 65504.0, 70000.0, -1e6, 6.1e-5, 5.9e-5, 1e-8, -3e-6, 1.0009765625, 1.00048828125,
                        np.inf, -np.inf, 3.3895314e38], dtype=np.float32)
    n = min(special.size, flat.size)
    flat[:n] = special[:n]
    return a


@pytest.fixture()
def sample(tmp_path):
    rng = np.random.default_rng(11)
    tensors = {
        "w.f32": (_values(rng, (6, 40)), "F32"),
        "w.f16": (_values(rng, (5, 24)), "F16"),
        "w.bf16": (_values(rng, (7, 16)), "BF16"),
        "norm.weight": (_values(rng, (40,)), "BF16"),
        "empty": (np.zeros((0, 8), dtype=np.float32), "F16"),
    }
    path = tmp_path / "model.safetensors"
    st.save_file(str(path), tensors, metadata={"format": "pt", "note": 'quotes " and {braces}'})
    return str(path), tensors


def _stored_values(array, stored):
    """What the file holds, as float32."""
    if stored == "F32":
        return np.asarray(array, dtype=np.float32)
    dt = Dtype.F16 if stored == "F16" else Dtype.BF16
    return orc.to_f32(orc.to_dtype(array, ORC_DT[dt]), ORC_DT[dt])


def _bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a


def test_parser_reads_header(sample):
    path, tensors = sample
    p = st.SafetensorsParser(path)
    assert sorted(p.get_tensor_names()) == sorted(tensors)
    for name, (array, stored) in tensors.items():
        assert p.get_shape(name) == array.shape and p.get_data_type(name) == stored
        assert p.byte_size(name) == array.size * (4 if stored == "F32" else 2)
    with pytest.raises(KeyError):
        p.get_shape("missing")
    with pytest.raises(ValueError):
        p["w.f32"].view(0, 10 ** 6)
    p.close()


@pytest.mark.parametrize("target", [Dtype.F32, Dtype.F16, Dtype.BF16])
def test_conversions_follow_the_loader_rules(sample, target):
    """Every file dtype -> every tensor dtype equals the oracle's conversion (fp16: round to
    nearest even, flush below the smallest normal, saturate to inf; bf16: round to nearest
    even) applied to the stored values."""
    path, tensors = sample
    p = st.SafetensorsParser(path)
    for name, (array, stored) in tensors.items():
        t = st.tensor(p[name], target)
        want = orc.to_dtype(_stored_values(array, stored), ORC_DT[target])
        assert t.shape == array.shape and t.dtype == target
        np.testing.assert_array_equal(_bits(t.host), _bits(np.asarray(want).reshape(array.shape)), err_msg=f"{name} -> {target}")
    keep = st.tensor(p["w.bf16"])
    assert keep.dtype == Dtype.BF16
    p.close()


def test_concat_and_slice(sample):
    path, tensors = sample
    p = st.SafetensorsParser(path)
    both = st.concat([p["w.bf16"], p["w.bf16"]], Dtype.F16)
    one = st.tensor(p["w.bf16"], Dtype.F16)
    assert both.shape == (14, 16)
    np.testing.assert_array_equal(both.host, np.concatenate([one.host, one.host]))
    rows = st.slice_rows(p["w.f32"], 2, 5, Dtype.BF16)
    np.testing.assert_array_equal(rows.host, st.tensor(p["w.f32"], Dtype.BF16).host[2:5])
    assert st.slice_rows(p["w.f32"], 3, 3, Dtype.F32).shape == (0, 40)
    with pytest.raises(ValueError):
        st.slice_rows(p["w.f32"], 4, 9, Dtype.F32)
    with pytest.raises(ValueError):
        st.concat([p["w.bf16"], p["w.f16"]], Dtype.F32)
    p.close()


def _raw_file(path, header, data=b""):
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + data)


def test_malformed_files_are_rejected(tmp_path):
    path = str(tmp_path / "bad.safetensors")
    with open(path, "wb") as f:
        f.write(b"\x01\x02")
    with pytest.raises(ValueError):
        st.SafetensorsParser(path)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(ValueError):
        st.SafetensorsParser(path)
    _raw_file(path, [1, 2])
    with pytest.raises(ValueError):
        st.SafetensorsParser(path)
    _raw_file(path, {"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8)      # data cut short
    with pytest.raises(ValueError):
        st.SafetensorsParser(path)
    _raw_file(path, {"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}}, b"\0" * 16)     # size != shape
    with pytest.raises(ValueError):
        st.SafetensorsParser(path).byte_size("t")
    _raw_file(path, {"t": {"dtype": "I64", "shape": [2], "data_offsets": [0, 16]}}, b"\0" * 16)
    with pytest.raises(ValueError):
        st.SafetensorsParser(path).byte_size("t")


def _tiny_llama(tmp_path, blocks=2, d=32, kv=16, ffn=48, vocab=50, shards=2):
    rng = np.random.default_rng(5)
    names = {"model.embed_tokens.weight": (vocab, d), "model.norm.weight": (d,)}
    for i in range(blocks):
        p = f"model.layers.{i}."
        names.update({p + "input_layernorm.weight": (d,), p + "post_attention_layernorm.weight": (d,),
                      p + "self_attn.q_proj.weight": (d, d), p + "self_attn.k_proj.weight": (kv, d),
                      p + "self_attn.v_proj.weight": (kv, d), p + "self_attn.o_proj.weight": (d, d),
                      p + "mlp.gate_proj.weight": (ffn, d), p + "mlp.up_proj.weight": (ffn, d),
                      p + "mlp.down_proj.weight": (d, ffn)})
    values = {k: rng.standard_normal(s).astype(np.float32) * 0.05 for k, s in names.items()}
    keys = sorted(values)
    for s in range(shards):
        part = {k: (values[k], "BF16") for k in keys[s::shards]}
        st.save_file(str(tmp_path / f"model-{s + 1:05d}-of-{shards:05d}.safetensors"), part)
    return values


def test_checkpoint_directory_and_llama_key_map(tmp_path):
    values = _tiny_llama(tmp_path)
    ckpt = st.Checkpoint(str(tmp_path))
    assert "model.norm.weight" in ckpt and "nope" not in ckpt
    with pytest.raises(KeyError):
        ckpt["nope"]
    w = st.load_llama_weights(ckpt, 2, w_dtype=Dtype.BF16)
    assert w["lmHead"] is w["embedding"]                               # tied
    assert w["finalNorm"].dtype == Dtype.F32 and w["blocks"][0]["norm1"].dtype == Dtype.F32
    blk = w["blocks"][1]
    assert blk["gateValue"].shape == (96, 32) and blk["projK"].shape == (16, 32) and blk["out"].shape == (32, 48)
    gate = orc.to_dtype(values["model.layers.1.mlp.gate_proj.weight"], orc.BF16)
    up = orc.to_dtype(values["model.layers.1.mlp.up_proj.weight"], orc.BF16)
    np.testing.assert_array_equal(blk["gateValue"].host, np.concatenate([gate, up]))       # gate rows first
    # a 3-way column split reads only each rank's rows and reassembles to the same matrices
    parts = [st.load_llama_weights(ckpt, 2, shard=(r, 3)) for r in range(3)]
    np.testing.assert_array_equal(np.concatenate([p["lmHead"].host for p in parts]), w["embedding"].host)
    g = np.concatenate([p["blocks"][1]["gateValue"].host[: p["blocks"][1]["gateValue"].shape[0] // 2] for p in parts])
    u = np.concatenate([p["blocks"][1]["gateValue"].host[p["blocks"][1]["gateValue"].shape[0] // 2:] for p in parts])
    np.testing.assert_array_equal(np.concatenate([g, u]), blk["gateValue"].host)
    ckpt.close()
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError):
        st.Checkpoint(str(tmp_path / "empty"))


def _fnv(b):
    h = 1469598103934665603
    for x in bytes(b):
        h = ((h ^ x) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def _cpp_exe():
    from test_host_cpp import _build
    return _build("host_safetensors_test")


def _check_cpp_listing(out, path, tensors):
    p = st.SafetensorsParser(path)
    lines = [ln for ln in out.splitlines() if " | " in ln]
    assert len(lines) == len(tensors)
    for ln in lines:
        left, right = ln.split(" | ")
        name, stored, *shape = left.split()
        fields = right.split()
        assert stored == tensors[name][1] and tuple(int(s) for s in shape) == tensors[name][0].shape
        assert int(fields[0]) == p.byte_size(name)
        for target, got in zip((Dtype.F32, Dtype.F16, Dtype.BF16), fields[1:4]):
            want = st.tensor(p[name], target).host
            assert int(got, 16) == _fnv(np.ascontiguousarray(want).tobytes()), f"{name} -> {target}"
    p.close()


def test_cpp_parser_and_conversions_match_python(sample):
    path, tensors = sample
    r = subprocess.run([_cpp_exe(), path], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    _check_cpp_listing(r.stdout, path, tensors)
    bad = path + ".cut"
    with open(path, "rb") as f, open(bad, "wb") as g:
        g.write(f.read()[:64])
    r = subprocess.run([_cpp_exe(), bad], capture_output=True, text=True)
    assert r.returncode == 3 and "error:" in r.stdout


@pytest.mark.gpu
def test_cpp_load_to_device(sample, device):
    path, tensors = sample
    r = subprocess.run([_cpp_exe(), path, "--gpu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "MISMATCH" not in r.stdout and "concat ok slice ok" in r.stdout
    _check_cpp_listing(r.stdout, path, tensors)


@pytest.mark.gpu
def test_cpp_large_tensor_crosses_staging_parts(tmp_path, device):
    """A 40 MiB tensor spans five 8 MiB staging parts in each direction of conversion."""
    rng = np.random.default_rng(2)
    big = rng.standard_normal((2560, 4096)).astype(np.float32)
    path = str(tmp_path / "big.safetensors")
    st.save_file(path, {"big": (big, "F32")})
    r = subprocess.run([_cpp_exe(), path, "--gpu"], capture_output=True, text=True)
    assert r.returncode == 0 and "MISMATCH" not in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_checkpoint_weights_drive_a_linear(tmp_path, device):
    """gate_proj | up_proj of a synthetic checkpoint -> gateValue Linear - GatedMul(SiLU), recorded
    as one launch, against float64 over the stored bf16 values."""
    import vai_b200
    from vai_b200 import Epilogue, Tensor, nodes
    values = _tiny_llama(tmp_path, blocks=1, d=64, kv=32, ffn=96, vocab=40, shards=1)
    ckpt = st.Checkpoint(str(tmp_path))
    w = st.load_llama_weights(ckpt, 1)

    class Net(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__(w_default_dtype=Dtype.BF16)
            self.lin = nodes.LinearNode(in_dim=64, out_dim=192)
            self.input("in0") - self.lin - nodes.GatedMulNode(activation=Epilogue.SILU) - self.output("out0")

    net = Net()
    net.lin["weight"] = w["blocks"][0]["gateValue"]
    x = np.random.default_rng(1).standard_normal((3, 64)).astype(np.float32)
    got = net(Tensor.from_numpy(x)).to_numpy()
    assert net.lin.gate_fuse
    gate = orc.to_f32(orc.to_dtype(values["model.layers.0.mlp.gate_proj.weight"], orc.BF16), orc.BF16)
    up = orc.to_f32(orc.to_dtype(values["model.layers.0.mlp.up_proj.weight"], orc.BF16), orc.BF16)
    want = orc.linear_f64(x, np.concatenate([gate, up]), epilogue=orc.EPILOGUES["SILU"], gate_fuse=True)
    np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-5)
    ckpt.close()


# ---- the one real checkpoint the reference ships -------------------------------------------
# tests/golden/mnist_jroot_model.safetensors is a byte-for-byte copy of the reference's
# data/ckpts/mnist/jroot/model.safetensors (201 KB, fp32; the weights of its MNIST example,
# examples/mnist/main.cpp:167-169).  Not written by this repository's save_file, so it pins
# the two readers to a file produced elsewhere; the `safetensors` wheel is the referee.

MNIST = os.path.join(ROOT, "tests", "golden", "mnist_jroot_model.safetensors")
MNIST_SHAPES = {"conv1.bias": (32,), "conv1.weight": (32, 1, 3, 3), "conv2.bias": (64,), "conv2.weight": (64, 32, 3, 3),
                "fc.bias": (10,), "fc.weight": (10, 3136)}


def test_reference_checkpoint_python_reader_equals_the_safetensors_wheel():
    from safetensors.numpy import load_file
    theirs = load_file(MNIST)
    p = st.SafetensorsParser(MNIST)
    assert sorted(p.get_tensor_names()) == sorted(MNIST_SHAPES) == sorted(theirs)
    for name, shape in MNIST_SHAPES.items():
        assert p.get_shape(name) == shape and p.get_data_type(name) == "F32"
        mine = st.tensor(p[name], Dtype.F32).host
        assert mine.shape == shape
        assert mine.tobytes() == np.ascontiguousarray(theirs[name]).tobytes(), name
        # and the conversions of the real values follow the loader's rules
        for target in (Dtype.F16, Dtype.BF16):
            np.testing.assert_array_equal(st.tensor(p[name], target).host, orc.to_dtype(theirs[name], ORC_DT[target]))
    p.close()


def test_reference_checkpoint_cpp_reader_equals_python():
    from safetensors.numpy import load_file
    theirs = load_file(MNIST)
    r = subprocess.run([_cpp_exe(), MNIST], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    _check_cpp_listing(r.stdout, MNIST, {k: (v, "F32") for k, v in theirs.items()})
    # the F32 column of the listing is the checksum of the raw bytes the wheel returns
    for ln in r.stdout.splitlines():
        if " | " in ln:
            name = ln.split()[0]
            assert int(ln.split(" | ")[1].split()[1], 16) == _fnv(np.ascontiguousarray(theirs[name]).tobytes())


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 5, 16, 130])
def test_reference_checkpoint_fc_layer_on_gpu(rows, device):
    """The checkpoint's fc Linear ([10, 3136] + bias, fp32 as the MNIST example loads it) driven by
    both readers' tensors: weight-streaming kernel for up to 8 rows, exact fp32 tile kernel above."""
    from linear_check import BOUND_FP32, FP32, assert_close
    from safetensors.numpy import load_file

    import vai_b200
    from vai_b200 import Tensor, nodes
    theirs = load_file(MNIST)
    p = st.SafetensorsParser(MNIST)

    class Net(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__(w_default_dtype=Dtype.F32)
            self.fc = nodes.LinearNode(in_dim=3136, out_dim=10)
            self.input("in0") - self.fc - self.output("out0")

    net = Net()
    net.fc["weight"] = st.tensor(p["fc.weight"], Dtype.F32)
    net.fc["bias"] = st.tensor(p["fc.bias"], Dtype.F32)
    x = np.random.default_rng(rows).standard_normal((rows, 3136)).astype(np.float32)
    got = net(Tensor.from_numpy(x)).to_numpy()
    want = orc.linear_f64(x, theirs["fc.weight"], theirs["fc.bias"])
    assert net.fc.info.kernel == (nodes.KERNEL_GEMV if rows <= 8 else nodes.KERNEL_FMA_TILE)
    assert_close(got, want, FP32 if rows <= 8 else BOUND_FP32, f"mnist fc, {rows} rows")
    p.close()


def test_hostile_headers_are_rejected(tmp_path):
    """Offsets and shapes chosen so that a sum or a product would wrap: both readers refuse the
    file instead of reading outside the mapping (the reference reads through fread and cannot)."""
    path = str(tmp_path / "hostile.safetensors")
    big = 2 ** 64
    cases = [
        {"t": {"dtype": "F32", "shape": [1], "data_offsets": [big - 100, big - 96]}},          # start_of_data + end wraps
        {"t": {"dtype": "F32", "shape": [1], "data_offsets": [-8, -4]}},                        # negative offsets
        {"t": {"dtype": "F32", "shape": [1], "data_offsets": [-8, 0]}},
        {"t": {"dtype": "F32", "shape": [2 ** 31, 2 ** 31, 4], "data_offsets": [0, 16]}},       # 2^64 elements "= 0"
        {"t": {"dtype": "F32", "shape": [2 ** 40], "data_offsets": [0, 16]}},                   # axis beyond 32 bits
        {"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 18446744073709551632]}},       # 2^64 + 16: beyond uint64
    ]
    for i, header in enumerate(cases):
        _raw_file(path, header, b"\0" * 16)
        with pytest.raises(ValueError):
            parser = st.SafetensorsParser(path)
            parser.byte_size("t")
            parser.view("t")
        r = subprocess.run([_cpp_exe(), path], capture_output=True, text=True)
        assert r.returncode == 3 and "error:" in r.stdout, (i, r.stdout)
