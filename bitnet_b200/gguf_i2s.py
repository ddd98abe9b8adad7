"""GGUF files with I2_S tensors: writer, reader, the dummy-model generator and the loader that
feeds them to the B200 kernels.

Counterpart of the reference's Python conversion tools:

* `quantize_to_i2_s` - utils/convert-hf-to-gguf-bitnet.py:666-727 (also src/ggml-bitnet-mad.cpp:51-96):
  ternary weights -> packed bytes (code = weight + 1, 128-value blocks, byte p of a block holds
  values p, p+32, p+64, p+96 in bit pairs 6-7, 4-5, 2-3, 0-1) plus a 32-byte tail whose first
  four bytes are the f32 scale.
* `write_gguf` / `read_gguf` - the GGUF v3 container as the reference's converters emit it:
  I2_S tensors are stored with their logical shape [N, K] and N*K/4 + 32 bytes of data
  (utils/convert-hf-to-gguf-bitnet.py:1164-1206), `general.file_type` = 40 (:157-159).  The
  upstream `gguf` Python package does not know the fork's tensor types, so the container is
  written and parsed here; the numeric id of I2_S (36) is the one the fork's `ggml.h` is
  believed to use - that header is not part of the checkout, so the id is a parameter.
* `generate_dummy_model` - utils/generate-dummy-bitnet-model.py:36-103 (size table), :804-809
  (absmean ternarisation), :824-848 (tensor list): a random model of a named size written as
  an I2_S GGUF, from a seed.
* `load_gguf_model` - reads such a file into `bitnet_b200.model.Transformer`: q/k/v and gate/up
  are fused, their I2_S bytes re-tiled on the GPU (`bitnet_pack_from_i2s`), the tail scales
  become the BitLinear's `weight_scale`.

Host-side file handling is Python, as the reference's is; the re-tiling runs on the GPU.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

GGUF_MAGIC = 0x46554747          # "GGUF"
GGUF_VERSION = 3
ALIGNMENT = 32

GGML_TYPE_F32, GGML_TYPE_F16 = 0, 1
GGML_TYPE_I2_S = 36               # the llama.cpp fork's id for I2_S (unverified: its ggml.h is not in the checkout)
LLAMA_FTYPE_MOSTLY_I2_S = 40      # utils/convert-hf-to-gguf-bitnet.py:157-159

# value types of GGUF metadata
_T_U8, _T_I8, _T_U16, _T_I16, _T_U32, _T_I32, _T_F32, _T_BOOL, _T_STR, _T_ARR, _T_U64, _T_I64, _T_F64 = range(13)
_SCALAR_FMT = {_T_U8: "<B", _T_I8: "<b", _T_U16: "<H", _T_I16: "<h", _T_U32: "<I", _T_I32: "<i", _T_F32: "<f",
               _T_BOOL: "<?", _T_U64: "<Q", _T_I64: "<q", _T_F64: "<d"}

# Size table of the dummy-model generator (utils/generate-dummy-bitnet-model.py:36-103):
# name -> (hidden, intermediate, layers, heads); vocabulary 32002, no grouped-query attention.
DUMMY_MODEL_CONFIG = {
    "125M": (768, 3072, 11, 12), "350M": (1024, 3072, 24, 16), "1B": (2048, 3584, 24, 32),
    "1.5B": (1536, 9216, 28, 32), "2.7B": (3072, 7680, 24, 32), "3.8B": (3840, 8192, 24, 32),
    "7B": (4096, 12032, 32, 32), "13B": (5120, 13824, 40, 40), "30B": (6656, 16384, 60, 52),
    "70B": (8192, 24576, 80, 64), "100B": (8192, 45568, 72, 64),
}
DUMMY_VOCAB = 32002


# ----------------------------------------------------------------------------------------
# I2_S bytes
# ----------------------------------------------------------------------------------------
def quantize_to_i2_s(w: np.ndarray, override_scale: Optional[float] = None) -> np.ndarray:
    """Float matrix [N, K] whose entries are 0 or +-scale (or, with override_scale, already
    -1/0/+1) -> I2_S bytes, N*K/4 + 32 long (utils/convert-hf-to-gguf-bitnet.py:666-727)."""
    flat = np.asarray(w, dtype=np.float32).reshape(-1)
    n = flat.size
    if n % 128 != 0:
        raise ValueError("I2_S packs blocks of 128 values: N*K must be a multiple of 128")
    if override_scale is not None:
        scale = np.float32(override_scale)
        tern = flat
    else:
        nz = np.abs(flat[np.abs(flat) > 1e-6])
        scale = np.float32(nz[0]) if nz.size else np.float32(1e-5)     # the first non-zero magnitude, as the C quantiser
        tern = np.clip(np.round(flat * (np.float32(1.0) / scale)), -1, 1)
    return pack_ternary_i2_s(tern, scale)


def pack_ternary_i2_s(tern: np.ndarray, scale) -> np.ndarray:
    """Ternary values (any shape, -1/0/+1) and a scale -> I2_S bytes."""
    t = np.asarray(tern).reshape(-1)
    n = t.size
    code = np.ones(n, dtype=np.uint8)
    code[t > 0.5] = 2
    code[t < -0.5] = 0
    blk = code.reshape(n // 128, 4, 32)
    packed = (blk[:, 0] << 6) | (blk[:, 1] << 4) | (blk[:, 2] << 2) | blk[:, 3]
    out = np.zeros(n // 4 + 32, dtype=np.uint8)
    out[: n // 4] = packed.reshape(-1)
    out[n // 4: n // 4 + 4] = np.frombuffer(np.float32(scale).tobytes(), dtype=np.uint8)
    return out


def i2_s_scale(buf: np.ndarray, n_values: int) -> np.float32:
    return np.frombuffer(np.asarray(buf[n_values // 4: n_values // 4 + 4], dtype=np.uint8).tobytes(), dtype=np.float32)[0]


def unpack_i2_s(buf: np.ndarray, n_rows: int, k: int) -> np.ndarray:
    """I2_S bytes -> ternary int8 [N, K] (code 3, which no writer emits, becomes +2)."""
    n = n_rows * k
    b = np.asarray(buf[: n // 4], dtype=np.uint8).reshape(n // 128, 32)
    c = np.stack([(b >> 6) & 3, (b >> 4) & 3, (b >> 2) & 3, b & 3], axis=1)
    return (c.reshape(n_rows, k).astype(np.int8) - 1)


def weight_quant(w: np.ndarray) -> np.ndarray:
    """absmean fake quantisation of the converters (utils/generate-dummy-bitnet-model.py:804-809):
    s = 1 / max(mean|W|, 1e-5); result = clamp(round(W s), -1, 1) / s."""
    w = np.asarray(w, dtype=np.float32)
    s = np.float32(1.0) / np.maximum(np.abs(w).mean(dtype=np.float32), np.float32(1e-5))
    return (np.clip(np.rint(w * s), -1, 1) / s).astype(np.float32)


# ----------------------------------------------------------------------------------------
# the container
# ----------------------------------------------------------------------------------------
def _gguf_str(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _kv_value(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<I", _T_BOOL) + struct.pack("<?", v)
    if isinstance(v, int):
        return struct.pack("<I", _T_U32) + struct.pack("<I", v) if 0 <= v < 2 ** 32 else struct.pack("<I", _T_I64) + struct.pack("<q", v)
    if isinstance(v, float):
        return struct.pack("<I", _T_F32) + struct.pack("<f", v)
    if isinstance(v, str):
        return struct.pack("<I", _T_STR) + _gguf_str(v)
    if isinstance(v, (list, tuple)):
        if all(isinstance(x, str) for x in v):
            return struct.pack("<IIQ", _T_ARR, _T_STR, len(v)) + b"".join(_gguf_str(x) for x in v)
        if all(isinstance(x, int) for x in v):
            return struct.pack("<IIQ", _T_ARR, _T_I32, len(v)) + struct.pack(f"<{len(v)}i", *v)
        return struct.pack("<IIQ", _T_ARR, _T_F32, len(v)) + struct.pack(f"<{len(v)}f", *[float(x) for x in v])
    raise TypeError(f"unsupported metadata value {type(v)}")


@dataclass
class TensorEntry:
    name: str
    shape: Tuple[int, ...]           # logical shape, outermost first (as NumPy)
    ggml_type: int
    data: np.ndarray                 # raw bytes (uint8) for I2_S, typed array otherwise


def _raw_bytes(t: TensorEntry) -> np.ndarray:
    return np.ascontiguousarray(t.data).view(np.uint8).reshape(-1)


def write_gguf(path: str, metadata: Dict[str, object], tensors: Sequence[TensorEntry]) -> None:
    """Writes a GGUF v3 file: header, metadata, tensor infos (dimensions innermost first), then
    the 32-byte aligned tensor data in the given order."""
    head = struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(tensors), len(metadata))
    kv = b"".join(_gguf_str(k) + _kv_value(v) for k, v in metadata.items())
    infos, offset, sizes = [], 0, []
    for t in tensors:
        nbytes = _raw_bytes(t).size
        dims = tuple(reversed(t.shape))
        infos.append(_gguf_str(t.name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims) +
                     struct.pack("<IQ", t.ggml_type, offset))
        sizes.append(nbytes)
        offset += (nbytes + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT
    with open(path, "wb") as f:
        f.write(head)
        f.write(kv)
        f.write(b"".join(infos))
        f.write(b"\0" * ((-f.tell()) % ALIGNMENT))
        for t, nbytes in zip(tensors, sizes):
            f.write(_raw_bytes(t).tobytes())
            f.write(b"\0" * ((-nbytes) % ALIGNMENT))


def _tensor_nbytes(ggml_type: int, shape: Tuple[int, ...], i2s_type: int) -> int:
    n = int(np.prod(shape)) if shape else 1
    if ggml_type == GGML_TYPE_F32:
        return 4 * n
    if ggml_type == GGML_TYPE_F16:
        return 2 * n
    if ggml_type == i2s_type:
        return n // 4 + 32
    raise ValueError(f"tensor type {ggml_type} is not handled by this reader")


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        v = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += struct.calcsize(fmt)
        return v if len(v) > 1 else v[0]

    def string(self) -> str:
        n = self.take("<Q")
        s = bytes(self.buf[self.pos: self.pos + n]).decode("utf-8")
        self.pos += n
        return s

    def value(self, vtype: int):
        if vtype == _T_STR:
            return self.string()
        if vtype == _T_ARR:
            et, n = self.take("<I"), self.take("<Q")
            return [self.value(et) for _ in range(n)]
        return self.take(_SCALAR_FMT[vtype])


def read_gguf(path: str, i2s_type: int = GGML_TYPE_I2_S):
    """Returns (metadata dict, {name: TensorEntry}); tensor data are views of a memory map."""
    buf = np.memmap(path, dtype=np.uint8, mode="r")
    c = _Cursor(buf)
    magic, version, n_tensors, n_kv = c.take("<I"), c.take("<I"), c.take("<Q"), c.take("<Q")
    if magic != GGUF_MAGIC or version not in (2, 3):
        raise ValueError("not a GGUF v2/v3 file")
    meta = {}
    for _ in range(n_kv):
        key = c.string()
        meta[key] = c.value(c.take("<I"))
    infos = []
    for _ in range(n_tensors):
        name = c.string()
        nd = c.take("<I")
        dims = [c.take("<Q") for _ in range(nd)]
        ttype, off = c.take("<I"), c.take("<Q")
        infos.append((name, tuple(reversed(dims)), ttype, off))
    align = int(meta.get("general.alignment", ALIGNMENT))
    base = (c.pos + align - 1) // align * align
    out = {}
    for name, shape, ttype, off in infos:
        nbytes = _tensor_nbytes(ttype, shape, i2s_type)
        raw = buf[base + off: base + off + nbytes]
        if ttype == GGML_TYPE_F32:
            data = raw.view(np.float32).reshape(shape)
        elif ttype == GGML_TYPE_F16:
            data = raw.view(np.float16).reshape(shape)
        else:
            data = raw
        out[name] = TensorEntry(name, shape, ttype, data)
    return meta, out


# ----------------------------------------------------------------------------------------
# dummy models
# ----------------------------------------------------------------------------------------
def _seed_for(seed: int, name: str) -> int:
    h = 1469598103934665603
    for ch in f"{seed}:{name}".encode():
        h = ((h ^ ch) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h & 0x7FFFFFFF


def dummy_tensor_list(hidden: int, inter: int, layers: int, heads: int, kv_heads: Optional[int] = None,
                      vocab: int = DUMMY_VOCAB) -> List[Tuple[str, Tuple[int, ...], bool]]:
    """(GGUF tensor name, shape, is a BitLinear weight) in the order the reference generator
    emits them (utils/generate-dummy-bitnet-model.py:824-848; rotary inv_freq is dropped there
    too, :860-862), with the GGUF names of llama.cpp's BitNet architecture."""
    kv = (kv_heads or heads) * (hidden // heads)
    out = [("token_embd.weight", (vocab, hidden), False)]
    for i in range(layers):
        b = f"blk.{i}."
        out += [(b + "attn_norm.weight", (hidden,), False), (b + "ffn_down.weight", (hidden, inter), True),
                (b + "ffn_sub_norm.weight", (inter,), False), (b + "ffn_gate.weight", (inter, hidden), True),
                (b + "ffn_up.weight", (inter, hidden), True), (b + "ffn_norm.weight", (hidden,), False),
                (b + "attn_sub_norm.weight", (hidden,), False), (b + "attn_k.weight", (kv, hidden), True),
                (b + "attn_output.weight", (hidden, hidden), True), (b + "attn_q.weight", (hidden, hidden), True),
                (b + "attn_v.weight", (kv, hidden), True)]
    out.append(("output_norm.weight", (hidden,), False))
    return out


def generate_dummy_model(path: str, size: str = "125M", seed: int = 0, *, hidden: Optional[int] = None,
                         inter: Optional[int] = None, layers: Optional[int] = None, heads: Optional[int] = None,
                         kv_heads: Optional[int] = None, vocab: int = DUMMY_VOCAB, rope_theta: float = 10000.0,
                         norm_eps: float = 1e-5, i2s_type: int = GGML_TYPE_I2_S) -> Dict[str, object]:
    """Writes a random BitNet model as an I2_S GGUF: every BitLinear weight is drawn N(0,1) from
    a generator seeded by (seed, tensor name), absmean-ternarised (weight_quant) and packed with
    quantize_to_i2_s; embeddings are f16, norm weights f32 (what the reference's converter
    emits for an I2_S file).  `size` names a row of the reference's table; explicit dimensions
    override it (the benchmark's architectures are not in that table).  Returns the metadata."""
    if hidden is None:
        hidden, inter, layers, heads = DUMMY_MODEL_CONFIG[size]
    kvh = kv_heads or heads
    meta = {
        "general.architecture": "bitnet", "general.name": f"dummy-{size}", "general.file_type": LLAMA_FTYPE_MOSTLY_I2_S,
        "general.alignment": ALIGNMENT, "bitnet.block_count": layers, "bitnet.context_length": 4096,
        "bitnet.embedding_length": hidden, "bitnet.feed_forward_length": inter, "bitnet.attention.head_count": heads,
        "bitnet.attention.head_count_kv": kvh, "bitnet.rope.freq_base": float(rope_theta),
        "bitnet.attention.layer_norm_rms_epsilon": float(norm_eps), "bitnet.vocab_size": vocab,
        "bitnet.rope.dimension_count": hidden // heads, "bitnet_b200.seed": seed,
    }
    tensors = []
    for name, shape, is_lin in dummy_tensor_list(hidden, inter, layers, heads, kvh, vocab):
        rng = np.random.default_rng(_seed_for(seed, name))
        if is_lin:
            w = weight_quant(rng.standard_normal(shape, dtype=np.float32))
            tensors.append(TensorEntry(name, shape, i2s_type, quantize_to_i2_s(w)))
        elif len(shape) == 2:
            tensors.append(TensorEntry(name, shape, GGML_TYPE_F16, rng.standard_normal(shape, dtype=np.float32).astype(np.float16)))
        else:
            # norm weights near one (the reference draws N(0,1); that makes no difference to a
            # throughput benchmark and a better conditioned model for parity checks)
            tensors.append(TensorEntry(name, shape, GGML_TYPE_F32, (1.0 + 0.1 * rng.standard_normal(shape)).astype(np.float32)))
    write_gguf(path, meta, tensors)
    return meta


# ----------------------------------------------------------------------------------------
# GGUF -> the kernel model
# ----------------------------------------------------------------------------------------
def model_args_from_gguf(meta: Dict[str, object]):
    from .config import ModelArgs

    arch = meta.get("general.architecture", "bitnet")
    g = lambda k, d=None: meta.get(f"{arch}.{k}", d)
    heads = int(g("attention.head_count"))
    return ModelArgs(dim=int(g("embedding_length")), n_layers=int(g("block_count")), n_heads=heads,
                     n_kv_heads=int(g("attention.head_count_kv", heads)), vocab_size=int(g("vocab_size")),
                     ffn_dim=int(g("feed_forward_length")), norm_eps=float(g("attention.layer_norm_rms_epsilon", 1e-5)),
                     rope_theta=float(g("rope.freq_base", 10000.0)), use_kernel=True, tie_embeddings=True)


def load_gguf_model(path: str, device="cuda", max_seq_len: int = 4096, rope_interleave: bool = True,
                    i2s_type: int = GGML_TYPE_I2_S):
    """Reads an I2_S GGUF into a `bitnet_b200.model.Transformer` on `device`.  q/k/v and gate/up
    are fused as gpu/convert_safetensors.py:61-84 fuses them; with rope_interleave the q and k
    rows go from the half-split rotary order of GGUF / Hugging Face files to the adjacent-pair
    order the decode kernels rotate (gpu/convert_safetensors.py:43-47)."""
    import torch

    from . import pack_weight
    from .model import Transformer, rope_table

    meta, tensors = read_gguf(path, i2s_type)
    args = model_args_from_gguf(meta)
    with torch.device("meta"):
        model = Transformer(args, max_seq_len)
    model = model.to_empty(device=device)
    D = args.head_dim

    def packed(name: str, n_heads_perm: int = 0):
        t = tensors[name]
        n, k = t.shape
        if t.ggml_type != i2s_type:
            raise ValueError(f"{name}: expected an I2_S tensor")
        scale = torch.tensor(float(i2_s_scale(t.data, n * k)), dtype=torch.bfloat16, device=device)
        if n_heads_perm and rope_interleave:
            # permuting rows of packed bytes means re-packing: unpack on the host, permute, pack on the GPU
            q = torch.from_numpy(unpack_i2_s(np.asarray(t.data), n, k)).to(device)
            q = q.view(n_heads_perm, 2, D // 2, k).transpose(1, 2).reshape(n, k).contiguous()
            return pack_weight.convert_weight_int8_to_int2(q), scale
        raw = torch.from_numpy(np.ascontiguousarray(t.data[: n * k // 4])).to(device)
        return pack_weight.convert_i2s_to_w2t(raw, n, k), scale

    def load_fused(lin, names_perm):
        parts, scales = zip(*(packed(nm, perm) for nm, perm in names_perm))
        lin.weight.data = torch.cat(parts, dim=0) if len(parts) > 1 else parts[0]
        ws = torch.zeros(4, dtype=torch.bfloat16, device=device)
        for i, s in enumerate(scales):
            ws[i] = s
        lin.weight_scale.data = ws
        lin.scale_f32 = ws[: len(lin.segments)].float().contiguous()

    def dense(name, dtype=torch.bfloat16):
        return torch.from_numpy(np.asarray(tensors[name].data).astype(np.float32)).to(device).to(dtype)

    model.tok_embeddings.weight.data = dense("token_embd.weight")
    if "output.weight" in tensors:
        model.output.weight.data = dense("output.weight")
        model.args.tie_embeddings = False
    else:
        model.output.weight = model.tok_embeddings.weight
    model.norm.weight.data = dense("output_norm.weight")
    for i, layer in enumerate(model.layers):
        b = f"blk.{i}."
        att, ff = layer.attention, layer.feed_forward
        load_fused(att.wqkv, [(b + "attn_q.weight", args.n_heads), (b + "attn_k.weight", args.n_kv_heads),
                              (b + "attn_v.weight", 0)])
        load_fused(att.wo, [(b + "attn_output.weight", 0)])
        load_fused(ff.w13, [(b + "ffn_gate.weight", 0), (b + "ffn_up.weight", 0)])
        load_fused(ff.w2, [(b + "ffn_down.weight", 0)])
        layer.attention_norm.weight.data = dense(b + "attn_norm.weight")
        layer.ffn_norm.weight.data = dense(b + "ffn_norm.weight")
        att.attn_sub_norm.weight.data = dense(b + "attn_sub_norm.weight")
        ff.ffn_sub_norm.weight.data = dense(b + "ffn_sub_norm.weight")
    model.rope = rope_table(D, max_seq_len, args.rope_theta, device)
    return model


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description="write a random BitNet model as an I2_S GGUF")
    ap.add_argument("--size", default="125M", choices=sorted(DUMMY_MODEL_CONFIG))
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--outfile", required=True)
    a = ap.parse_args()
    print(generate_dummy_model(a.outfile, a.size, a.seed))
