"""`.nnue` files: writing a trained model and reading a file back, either into
a float model or straight into the integer tensors of `QuantizedNet`.

File layout (all little endian), as the reference project's
model/utils/serialize.py:102-400 writes and reads it:

  u32 version, u32 network hash, u32 len + description (utf-8)
  u32 feature-transformer hash
  FT bias            int16 [L1]
  per feature block: FT weights int16 (int8 for threat blocks) [rows, L1],
                     PSQT weights int32 [rows, psqt buckets]
  per layer-stack bucket: u32 layers hash, then for l1, l2, output:
                     bias int32 [out], weights int8 [out, inputs padded to 32]

A tensor of a type wider than one byte may be stored as the magic string
`COMPRESSED_LEB128`, a u32 byte count and signed LEB128 varints.  Values are
`round(float * scale)`; a value outside the symmetric range of the target type
is an error, never a silent clip (model/quantize.py:18-34,175-235 there).
The LEB128 coder here works on whole numpy arrays instead of a per-value loop.
"""

from __future__ import annotations

import io
import struct
from typing import BinaryIO

import numpy as np
import torch

from .quantize import QuantizationManager

VERSION = 0x6A448AFA
DEFAULT_DESCRIPTION = "Network trained with the https://github.com/official-stockfish/nnue-pytorch trainer."
LEB128_MAGIC = b"COMPRESSED_LEB128"


# ---- signed LEB128 on arrays -------------------------------------------------
def encode_leb128(values: np.ndarray) -> bytes:
    """Signed LEB128 of every element, concatenated."""
    v = np.asarray(values).astype(np.int64).ravel()
    n = v.size
    if n == 0:
        return b""
    # a value needs k groups of 7 bits when it fits a signed (7k)-bit integer
    groups = np.ones(n, dtype=np.int64)
    for k in range(1, 10):
        lim = np.int64(1) << (7 * k - 1)
        groups = np.where((v >= lim) | (v < -lim), k + 1, groups)
    offsets = np.concatenate(([0], np.cumsum(groups)))
    out = np.zeros(offsets[-1], dtype=np.uint8)
    for k in range(int(groups.max())):
        sel = groups > k
        byte = ((v[sel] >> (7 * k)) & 0x7F).astype(np.uint8)
        more = (groups[sel] > k + 1).astype(np.uint8) << 7
        out[offsets[:-1][sel] + k] = byte | more
    return out.tobytes()


def decode_leb128(buf: bytes, count: int) -> np.ndarray:
    """The first `count` signed LEB128 values of `buf` as int64."""
    b = np.frombuffer(buf, dtype=np.uint8)
    ends = np.flatnonzero((b & 0x80) == 0)
    if ends.size < count:
        raise EOFError("LEB128 stream holds fewer values than expected")
    ends = ends[:count]
    starts = np.concatenate(([0], ends[:-1] + 1)) if count else np.zeros(0, dtype=np.int64)
    lengths = ends - starts + 1
    out = np.zeros(count, dtype=np.int64)
    for k in range(int(lengths.max()) if count else 0):
        sel = lengths > k
        out[sel] |= (b[starts[sel] + k].astype(np.int64) & 0x7F) << (7 * k)
    sign = (b[ends].astype(np.int64) & 0x40) != 0
    shift = 7 * lengths
    out = np.where(sign & (shift < 64), out | -(np.int64(1) << np.minimum(shift, 62)), out)
    return out


# ---- quantization of the export (model/quantize.py:18-34 of the reference) --------
def safe_convert(value: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """round(value) in `dtype`; raises when a value leaves [-max, max]."""
    lim = torch.iinfo(dtype).max
    r = value.round()
    bad = int(((r < -lim) | (r > lim)).sum())
    if bad:
        raise RuntimeError(
            f"Found {bad} out of bounds values when converting to target dtype {dtype}. "
            f"Min: {r.min().item()}, max: {r.max().item()}."
        )
    return r.to(dtype)


def layers_hash(l1: int, outs: tuple[int, int, int] = (32, 32, 1)) -> int:
    """Hash of the three fully connected layers behind an input slice of 2*l1."""
    prev = 0xEC42E90D ^ (l1 * 2)
    h = prev
    for out in outs:
        h = 0xCC03DAE4 + out
        h ^= prev >> 1
        h ^= (prev << 31) & 0xFFFFFFFF
        if out != 1:
            h = (h + 0x538D24C7) & 0xFFFFFFFF  # clipped ReLU follows
        prev = h
    return h & 0xFFFFFFFF


def _stack_layers(ls, bucket: int):
    """Float (weight, bias) of bucket `bucket` for l1 (factor folded in), l2 and output."""
    out = []
    for layer in (ls.l1, ls.l2, ls.output):
        o = layer.out_features
        w = layer.linear.weight.data[bucket * o : (bucket + 1) * o].detach().float().cpu()
        b = layer.linear.bias.data[bucket * o : (bucket + 1) * o].detach().float().cpu()
        f = getattr(layer, "factorized_linear", None)
        if f is not None:
            w = w + f.weight.data.detach().float().cpu()
            b = b + f.bias.data.detach().float().cpu()
        out.append((w, b, layer.layer_key))
    return out


class NNUEWriter:
    """`NNUEWriter(model).buf` holds the file's bytes."""

    def __init__(self, model, description: str | None = None, ft_compression: str = "none"):
        if ft_compression not in ("none", "leb128"):
            raise ValueError("Invalid compression method.")
        self.buf = bytearray()
        q: QuantizationManager = model.quantization
        scales = q.weight_scales_dict
        l1 = model.L1
        ls = model.layer_stacks
        fc = layers_hash(l1, (ls.l1.out_features, ls.l2.out_features, ls.output.out_features))
        feature_hash = model.input.HASH
        desc = (DEFAULT_DESCRIPTION if description is None else description).encode("utf-8")
        self._u32(VERSION)
        self._u32(fc ^ feature_hash ^ (l1 * 2))
        self._u32(len(desc))
        self.buf.extend(desc)
        self._u32(feature_hash ^ (l1 * 2))

        ft = model.input
        bias = ft.bias.data[:l1].detach().float().cpu()
        self._tensor(safe_convert(bias.mul(scales["ft_bias"]), torch.int16), ft_compression)
        export = ft.get_export_weights().detach().float().cpu()
        at = 0
        for f in ft.features:
            n = f.NUM_REAL_FEATURES
            dtype = getattr(f, "EXPORT_WEIGHT_DTYPE", torch.int16)
            seg = export[at : at + n]
            at += n
            w = safe_convert(seg[:, :l1].mul(scales["ft_weight"]), dtype)
            p = safe_convert(seg[:, l1:].mul(scales["ft_psqt_weight"]), torch.int32)
            self._tensor(w, ft_compression if dtype != torch.int8 else "none")
            self._tensor(p, ft_compression)

        for bucket in range(ls.count):
            self._u32(fc)
            for w, b, key in _stack_layers(ls, bucket):
                qb = safe_convert(b.mul(scales[f"{key}_bias"]), torch.int32)
                qw = safe_convert(w.mul(scales[f"{key}_weight"]), torch.int8)
                pad = (-qw.shape[1]) % 32  # inputs padded to a multiple of 32
                if pad:
                    qw = torch.nn.functional.pad(qw, (0, pad))
                self._tensor(qb, "none")
                self._tensor(qw, "none")

    def _u32(self, v: int) -> None:
        self.buf.extend(struct.pack("<I", v & 0xFFFFFFFF))

    def _tensor(self, t: torch.Tensor, compression: str) -> None:
        arr = t.contiguous().numpy().ravel()
        if compression == "none":
            self.buf.extend(arr.astype(arr.dtype.newbyteorder("<")).tobytes())
        else:
            enc = encode_leb128(arr)
            self.buf.extend(LEB128_MAGIC)
            self._u32(len(enc))
            self.buf.extend(enc)


class NNUEFile:
    """The integer tensors of a `.nnue` file, as stored.

    ft_bias int16 [L1]; ft_weight [rows, L1] (int16, or int8 for threat
    blocks, concatenated as int16); ft_psqt int32 [rows, P]; per bucket
    l1/l2/out weights int8 (padding stripped) and biases int32."""

    def __init__(self, f: BinaryIO, feature_blocks, l1: int, num_psqt_buckets: int = 8, num_ls_buckets: int = 8,
                 l2: int = 32, l3: int = 32, feature_hash: int | None = None):
        """feature_blocks: [(rows, numpy dtype of the stored weights)] in file order."""
        self.f = f
        self.L1, self.L2, self.L3, self.P, self.buckets = l1, l2, l3, num_psqt_buckets, num_ls_buckets
        fc = layers_hash(l1, (l2, l3, 1))
        self._expect(VERSION, "version")
        net_hash = self._u32()
        if feature_hash is not None and net_hash != (fc ^ feature_hash ^ (l1 * 2)):
            raise ValueError(f"Expected: {fc ^ feature_hash ^ (l1 * 2):x}, got: {net_hash:x}")
        self.description = f.read(self._u32()).decode("utf-8")
        ft_hash = self._u32()
        if feature_hash is not None and ft_hash != (feature_hash ^ (l1 * 2)):
            raise ValueError(f"Expected: {feature_hash ^ (l1 * 2):x}, got: {ft_hash:x}")
        self.ft_bias = self._tensor(np.int16, (l1,))
        ws, ps = [], []
        for rows, dtype in feature_blocks:
            ws.append(self._tensor(dtype, (rows, l1)).astype(np.int16))
            ps.append(self._tensor(np.int32, (rows, num_psqt_buckets)))
        self.ft_weight = np.concatenate(ws, axis=0)
        self.ft_psqt = np.concatenate(ps, axis=0)
        shapes = [(l2, l1), (l3, 2 * l2), (1, 2 * l2 + 2 * l3)]
        self.fc = []  # [bucket][layer] = (weight int8 [out, in], bias int32 [out])
        for _ in range(num_ls_buckets):
            self._expect(fc, "layers hash")
            layers = []
            for out, inp in shapes:
                b = self._tensor(np.int32, (out,))
                w = self._tensor(np.int8, (out, (inp + 31) // 32 * 32))[:, :inp]
                layers.append((np.ascontiguousarray(w), b))
            self.fc.append(layers)

    def _u32(self) -> int:
        d = self.f.read(4)
        if len(d) != 4:
            raise EOFError("Unexpected end of file")
        return struct.unpack("<I", d)[0]

    def _expect(self, want: int, what: str) -> None:
        got = self._u32()
        if got != want:
            raise ValueError(f"Expected: {want:x}, got: {got:x} ({what})")

    def _tensor(self, dtype, shape) -> np.ndarray:
        count = int(np.prod(shape))
        pos = self.f.tell()
        magic = self.f.read(len(LEB128_MAGIC))
        if magic == LEB128_MAGIC:
            nbytes = self._u32()
            d = self.f.read(nbytes)
            if len(d) != nbytes:
                raise EOFError("Unexpected end of file when reading compressed data.")
            return decode_leb128(d, count).astype(dtype).reshape(shape)
        self.f.seek(pos)
        size = count * np.dtype(dtype).itemsize
        d = self.f.read(size)
        if len(d) != size:
            raise EOFError("Unexpected end of file")
        return np.frombuffer(d, dtype=np.dtype(dtype).newbyteorder("<")).astype(dtype).reshape(shape)


def _blocks_of(ft) -> list[tuple[int, type]]:
    return [(f.NUM_REAL_FEATURES, np.int8 if getattr(f, "EXPORT_WEIGHT_DTYPE", torch.int16) == torch.int8 else np.int16)
            for f in ft.features]


class NNUEReader:
    """`NNUEReader(f, feature_name, config).model` is a float model holding the
    file's weights (factor layers zero), like the reference's reader."""

    def __init__(self, f: BinaryIO, feature_name: str, config=None):
        from .model import ModelConfig, NNUEModel

        config = config or ModelConfig()
        self.model = NNUEModel(feature_name, config)
        m = self.model
        nf = NNUEFile(f, _blocks_of(m.input), m.L1, m.num_psqt_buckets, m.num_ls_buckets, m.L2, m.L3, m.input.HASH)
        self.description, self.file = nf.description, nf
        s = m.quantization.weight_scales_dict
        with torch.no_grad():
            m.input.zero_virtual_weights()
            bias = torch.from_numpy(nf.ft_bias.astype(np.float32)) / s["ft_bias"]
            m.input.bias.data = torch.cat([bias, torch.zeros(m.num_psqt_buckets)])
            w = torch.from_numpy(nf.ft_weight.astype(np.float32)) / s["ft_weight"]
            p = torch.from_numpy(nf.ft_psqt.astype(np.float32)) / s["ft_psqt_weight"]
            m.input.load_export_weights(torch.cat([w, p], dim=1))
            ls = m.layer_stacks
            ls.l1.zero_virtual_weights()
            for bucket, layers in enumerate(nf.fc):
                for layer, (qw, qb) in zip((ls.l1, ls.l2, ls.output), layers):
                    o = layer.out_features
                    layer.linear.weight.data[bucket * o : (bucket + 1) * o] = (
                        torch.from_numpy(qw.astype(np.float32)) / s[f"{layer.layer_key}_weight"])
                    layer.linear.bias.data[bucket * o : (bucket + 1) * o] = (
                        torch.from_numpy(qb.astype(np.float32)) / s[f"{layer.layer_key}_bias"])


def save_nnue(model, path: str, description: str | None = None, ft_compression: str = "leb128") -> None:
    with open(path, "wb") as f:
        f.write(NNUEWriter(model, description, ft_compression).buf)


def load_quantized(path_or_file, feature_name: str, config=None, device="cuda"):
    """A `QuantizedNet` holding exactly the file's integers (no float round trip).
    The index lists it evaluates are those of the export layout: 11 planes per
    king bucket, 22528 rows for HalfKAv2_hm."""
    from .features import get_feature_cls
    from .model import ModelConfig
    from .quantized_eval import QuantizedNet

    config = config or ModelConfig()
    blocks = [(f.NUM_REAL_FEATURES, np.int8 if getattr(f, "EXPORT_WEIGHT_DTYPE", torch.int16) == torch.int8 else np.int16)
              for f in get_feature_cls(feature_name)]
    f = open(path_or_file, "rb") if isinstance(path_or_file, (str, bytes)) else path_or_file
    try:
        nf = NNUEFile(f, blocks, config.L1, 8, 8, config.L2, config.L3, None)
    finally:
        if isinstance(path_or_file, (str, bytes)):
            f.close()
    return QuantizedNet.from_integers(nf, QuantizationManager(config.quantize_config), torch.device(device))


def to_bytes(model, **kw) -> bytes:
    return bytes(NNUEWriter(model, **kw).buf)


def from_bytes(data: bytes, feature_name: str, config=None) -> NNUEReader:
    return NNUEReader(io.BytesIO(data), feature_name, config)
