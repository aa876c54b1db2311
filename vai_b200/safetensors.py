"""Weight ingest from safetensors checkpoints: the on-disk format of the Linear path's
largest operand.

Mirrors vAi's loader: `SafetensorsParser` / `SafetensorRef`
(vai/engine/safetensors-parser.h:18-56), `Checkpoint` over a directory of shards
(vai/engine/weights.h:30-64), `Tensor(ref, dtype)`, `concat` and `slice` with the
file-dtype conversions (vai/engine/tensor.cpp:183-312; BF16 is a file format there and a
tensor dtype here, so BF16 -> BF16 is a plain copy), and the Llama 3 key map
(models/production/llama3/meta-weights.h:23-68).

The file is memory-mapped; a tensor is a zero-copy view until it is converted.  `slice`
reads only the requested rows, which is how a rank of a column-split Linear ingests its
slab without touching the rest of the matrix."""
import json
import mmap
import os
import struct

import numpy as np

from .engine import Dtype, Tensor, bits_to_f32, f32_to_bf16_bits, f32_to_f16_bits

_FILE_DTYPES = {"F32": (np.float32, 4), "F16": (np.uint16, 2), "BF16": (np.uint16, 2)}


class SafetensorRef:
    """One tensor of one file: shape, file dtype and its bytes."""

    def __init__(self, parser, key):
        self.parser, self.key = parser, key

    def get_shape(self):
        return self.parser.get_shape(self.key)

    def get_data_type(self):
        return self.parser.get_data_type(self.key)

    def byte_size(self):
        return self.parser.byte_size(self.key)

    def view(self, byte_offset=0, byte_count=None):
        """Read-only array over the mapped bytes (uint16 bit patterns for F16 / BF16)."""
        return self.parser.view(self.key, byte_offset, byte_count)


class SafetensorsParser:
    """Header of a .safetensors file: 8-byte little-endian length, a JSON object
    name -> {dtype, shape, data_offsets}, then the data section."""

    def __init__(self, path):
        self.path = path
        self._file = open(path, "rb")
        size = os.fstat(self._file.fileno()).st_size
        head = self._file.read(8)
        if len(head) != 8:
            raise ValueError("Failed to read header length.")
        (n,) = struct.unpack("<Q", head)
        if 8 + n > size:
            raise ValueError("Failed to read header string.")
        try:
            root = json.loads(self._file.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise ValueError(f"JSON parse error: {e}") from None
        if not isinstance(root, dict):
            raise ValueError("Invalid Safetensors: root is not object")
        self.start_of_data = 8 + n
        self.tensors = {}
        for key, meta in root.items():
            if key == "__metadata__":
                continue
            if not isinstance(meta, dict):
                raise ValueError(f"Invalid tensor entry: {key}")
            try:
                begin, end = (int(v) for v in meta["data_offsets"])
                shape = tuple(int(s) for s in meta["shape"])
            except (KeyError, TypeError, ValueError):
                raise ValueError(f"Invalid tensor entry: {key}") from None
            if not 0 <= begin <= end or end > size - self.start_of_data:
                raise ValueError(f"Tensor data runs past the end of the file: {key}")
            if any(s < 0 or s > 0xFFFFFFFF for s in shape):
                raise ValueError(f"Invalid tensor entry (axis out of range): {key}")
            self.tensors[key] = (str(meta["dtype"]), shape, begin, end)
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None
        self._file.close()

    def get_tensor_names(self):
        return list(self.tensors)

    def __contains__(self, key):
        return key in self.tensors

    def __getitem__(self, key):
        return SafetensorRef(self, key)

    def _meta(self, key):
        try:
            return self.tensors[key]
        except KeyError:
            raise KeyError(f"Tensor key not found: {key}") from None

    def get_shape(self, key):
        return self._meta(key)[1]

    def get_data_type(self, key):
        return self._meta(key)[0]

    def byte_size(self, key):
        dtype, shape, begin, end = self._meta(key)
        if dtype not in _FILE_DTYPES:
            raise ValueError(f"Unsupported dtype: {dtype}")
        elems = 1
        for axis in shape:          # Python integers: the product cannot wrap
            elems *= axis
        if end - begin != elems * _FILE_DTYPES[dtype][1]:
            raise ValueError(f"Data size mismatch for {dtype} tensor.")
        return end - begin

    def view(self, key, byte_offset=0, byte_count=None):
        total = self.byte_size(key)
        dtype, _, begin, _ = self._meta(key)
        count = total - byte_offset if byte_count is None else byte_count
        if byte_offset < 0 or count < 0 or byte_offset + count > total:
            raise ValueError("Tensor read runs past the end of the tensor.")
        np_dtype, esz = _FILE_DTYPES[dtype]
        if byte_offset % esz or count % esz:
            raise ValueError("Tensor read does not fall on element boundaries.")
        return np.frombuffer(self._map, dtype=np_dtype, count=count // esz, offset=self.start_of_data + begin + byte_offset)


class Checkpoint:
    """Every *.safetensors under a directory, addressed by tensor name."""

    def __init__(self, directory):
        self.shards = []
        self.owner = {}
        for name in sorted(os.listdir(directory)):
            if not name.endswith(".safetensors"):
                continue
            shard = SafetensorsParser(os.path.join(directory, name))
            self.shards.append(shard)
            for key in shard.get_tensor_names():
                self.owner.setdefault(key, shard)
        if not self.owner:
            raise FileNotFoundError(f"no *.safetensors under {directory}")

    def __contains__(self, key):
        return key in self.owner

    def __getitem__(self, key):
        if key not in self.owner:
            raise KeyError(f"checkpoint has no tensor {key}")
        return self.owner[key][key]

    def close(self):
        for s in self.shards:
            s.close()


def _dtype_of_file(stored):
    return {"F32": Dtype.F32, "F16": Dtype.F16, "BF16": Dtype.BF16}[stored]


def convert_stored(raw, stored, target):
    """File values -> the array a tensor of dtype `target` holds (float32, or uint16 bit
    patterns).  16-bit -> 16-bit of the other kind goes through fp32, which holds both
    exactly, and rounds once to nearest even; fp16 results below the smallest normal flush
    to zero and overflow goes to inf (tensor.cpp:46-70)."""
    target = Dtype(target)
    if _dtype_of_file(stored) == target:
        return np.array(raw)            # copy out of the mapping
    vals = np.asarray(raw, dtype=np.float32) if stored == "F32" else bits_to_f32(raw, _dtype_of_file(stored))
    if target == Dtype.F32:
        return np.ascontiguousarray(vals, dtype=np.float32)
    return f32_to_f16_bits(vals) if target == Dtype.F16 else f32_to_bf16_bits(vals)


def _host_tensor(shape, dtype, host):
    t = Tensor(shape, dtype)
    t.host = host.reshape(shape)
    return t


def tensor(ref, dtype=None):
    """Tensor(ref, dtype): the whole file tensor as `dtype` (None keeps the file's)."""
    stored = ref.get_data_type()
    target = _dtype_of_file(stored) if dtype is None or Dtype(dtype) == Dtype.NONE else Dtype(dtype)
    return _host_tensor(ref.get_shape(), target, convert_stored(ref.view(), stored, target))


def concat(refs, dtype):
    """File tensors stacked along the leading axis (gate_proj over up_proj -> the
    [2H, K] weight of a gate|value Linear)."""
    refs = list(refs)
    if not refs or Dtype(dtype) == Dtype.NONE:
        raise ValueError("concat needs tensors and a target dtype")
    stored = refs[0].get_data_type()
    tail = refs[0].get_shape()[1:]
    parts = []
    for r in refs:
        if r.get_data_type() != stored or r.get_shape()[1:] != tail or not r.get_shape():
            raise ValueError("concat: tensors differ in dtype or trailing shape")
        parts.append(convert_stored(r.view(), stored, dtype).reshape(r.get_shape()))
    out = np.concatenate(parts, axis=0)
    return _host_tensor(out.shape, Dtype(dtype), out)


def slice_rows(ref, begin, end, dtype):
    """Rows [begin, end) of the leading axis; only those bytes are read."""
    shape = ref.get_shape()
    if not shape or not 0 <= begin <= end <= shape[0]:
        raise ValueError("slice: row range out of bounds")
    stored = ref.get_data_type()
    row_bytes = ref.byte_size() // shape[0] if shape[0] else 0
    raw = ref.view(begin * row_bytes, (end - begin) * row_bytes)
    new_shape = (end - begin,) + tuple(shape[1:])
    return _host_tensor(new_shape, Dtype(dtype), convert_stored(raw, stored, dtype))


def load_llama_weights(ckpt, n_blocks, w_dtype=Dtype.BF16, norm_dtype=Dtype.F32, shard=None):
    """The Linear and norm parameters of a Llama-3-style checkpoint, keyed as the
    reference wires them (meta-weights.h:23-68): per block norm1 / norm2 scales, projQ,
    projK, projV, projOut, gateValue = gate_proj over up_proj, out = down_proj; finalNorm;
    embedding, and lmHead aliasing the embedding (tied).

    shard = (rank, world) keeps only this rank's rows of the column-split layers
    (gateValue and lmHead), read with slice_rows so the other ranks' bytes stay on disk."""
    from .sharded import shard_rows
    out = {"blocks": []}
    out["embedding"] = tensor(ckpt["model.embed_tokens.weight"], w_dtype)
    for i in range(n_blocks):
        p = f"model.layers.{i}."
        blk = {
            "norm1": tensor(ckpt[p + "input_layernorm.weight"], norm_dtype),
            "norm2": tensor(ckpt[p + "post_attention_layernorm.weight"], norm_dtype),
            "projQ": tensor(ckpt[p + "self_attn.q_proj.weight"], w_dtype),
            "projK": tensor(ckpt[p + "self_attn.k_proj.weight"], w_dtype),
            "projV": tensor(ckpt[p + "self_attn.v_proj.weight"], w_dtype),
            "projOut": tensor(ckpt[p + "self_attn.o_proj.weight"], w_dtype),
            "out": tensor(ckpt[p + "mlp.down_proj.weight"], w_dtype),
        }
        gate, up = ckpt[p + "mlp.gate_proj.weight"], ckpt[p + "mlp.up_proj.weight"]
        if shard is None:
            blk["gateValue"] = concat([gate, up], w_dtype)
        else:
            begin, count = shard_rows(gate.get_shape()[0], shard[1], shard[0])
            g = slice_rows(gate, begin, begin + count, w_dtype)
            u = slice_rows(up, begin, begin + count, w_dtype)
            both = np.concatenate([g.host, u.host], axis=0)
            blk["gateValue"] = _host_tensor(both.shape, Dtype(w_dtype), both)
        out["blocks"].append(blk)
    out["finalNorm"] = tensor(ckpt["model.norm.weight"], norm_dtype)
    if shard is None:
        out["lmHead"] = out["embedding"]            # tied: the same storage
    else:
        emb = ckpt["model.embed_tokens.weight"]
        begin, count = shard_rows(emb.get_shape()[0], shard[1], shard[0])
        out["lmHead"] = slice_rows(emb, begin, begin + count, w_dtype)
    return out


def save_file(path, tensors, metadata=None):
    """Writes {name: (array, "F32" | "F16" | "BF16")} as a .safetensors file; arrays are
    float32 values, converted on the way out.  Used by the tests and for exporting
    synthetic checkpoints of the benchmark shapes."""
    header, blobs, pos = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, (array, stored) in tensors.items():
        a = np.asarray(array, dtype=np.float32)
        raw = a if stored == "F32" else (f32_to_f16_bits(a) if stored == "F16" else f32_to_bf16_bits(a))
        blob = np.ascontiguousarray(raw).tobytes()
        header[name] = {"dtype": stored, "shape": list(a.shape), "data_offsets": [pos, pos + len(blob)]}
        blobs.append(blob)
        pos += len(blob)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for b in blobs:
            f.write(b)
