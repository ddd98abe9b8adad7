"""Checkpoint and GGUF conversion: host logic against golden vectors from the reference's own
converters (tests/golden/ref_converters.npz) and the NumPy oracle; the GPU parts are marked."""
import os

import numpy as np
import pytest
import torch

from oracle import np_oracle as O


def _golden(golden_dir):
    return np.load(os.path.join(golden_dir, "ref_converters.npz"))


def test_quantize_to_i2_s_matches_reference_converter(golden_dir, port_lib):
    from bitnet_b200 import gguf_i2s as G

    g = _golden(golden_dir)
    for i in range(3):
        wq = g[f"wq_{i}"]
        got = G.quantize_to_i2_s(wq)
        assert np.array_equal(got, g[f"i2s_{i}"])                        # the reference's Python converter
        assert np.array_equal(got, port_lib.quantize_i2_s(wq))           # ... and its C quantiser (via the port)
        tern, ov = g[f"tern_{i}"], 0.625 + i
        got = G.quantize_to_i2_s(tern, override_scale=ov)
        assert np.array_equal(got, g[f"i2s_override_{i}"])
        assert np.array_equal(G.unpack_i2_s(got, *tern.shape), tern.astype(np.int8))
        assert G.i2_s_scale(got, tern.size) == np.float32(ov)
        assert np.array_equal(got, O.i2s_pack(tern.astype(np.int8), ov))


def test_rope_row_permutation_matches_reference(golden_dir):
    from bitnet_b200.convert_checkpoint import rope_rows_to_interleaved

    g = _golden(golden_dir)
    got = rope_rows_to_interleaved(torch.from_numpy(g["rope_in"]), n_heads=4)
    assert np.array_equal(got.numpy(), g["rope_out"])


def test_weight_quant_equals_oracle_ternarize():
    from bitnet_b200 import gguf_i2s as G

    w = np.random.default_rng(5).standard_normal((48, 256)).astype(np.float32)
    q, s = O.ternarize(w)
    wq = G.weight_quant(w)
    assert np.array_equal(np.sign(wq).astype(np.int8), q)
    nz = np.abs(wq[wq != 0])
    assert np.allclose(nz, s, rtol=1e-6)


def test_gguf_container_round_trip(tmp_path):
    from bitnet_b200 import gguf_i2s as G

    path = str(tmp_path / "m.gguf")
    meta = G.generate_dummy_model(path, hidden=256, inter=384, layers=2, heads=4, kv_heads=2, vocab=512, seed=3,
                                  size="custom")
    meta2, tensors = G.read_gguf(path)
    assert meta2["general.file_type"] == 40 and meta2["general.architecture"] == "bitnet"
    for k, v in meta.items():        # floats are stored as f32
        assert meta2[k] == (pytest.approx(v, rel=1e-6) if isinstance(v, float) else v)
    names = [n for n, _, _ in G.dummy_tensor_list(256, 384, 2, 4, 2, 512)]
    assert list(tensors) == names and len(names) == 2 * 11 + 2
    t = tensors["blk.1.ffn_gate.weight"]
    assert t.shape == (384, 256) and t.ggml_type == G.GGML_TYPE_I2_S and t.data.size == 384 * 256 // 4 + 32
    # the same seed gives the same bytes; the ternary content follows the absmean rule
    rng = np.random.default_rng(G._seed_for(3, "blk.1.ffn_gate.weight"))
    w = rng.standard_normal((384, 256), dtype=np.float32)
    q, s = O.ternarize(w)
    assert np.array_equal(G.unpack_i2_s(np.asarray(t.data), 384, 256), q)
    assert np.isclose(G.i2_s_scale(np.asarray(t.data), 384 * 256), s, rtol=1e-6)
    assert tensors["token_embd.weight"].data.dtype == np.float16 and tensors["output_norm.weight"].data.dtype == np.float32
    # the reference's size table
    assert G.DUMMY_MODEL_CONFIG["100B"] == (8192, 45568, 72, 64) and G.DUMMY_VOCAB == 32002


def test_unpack_offline_uint8():
    from bitnet_b200.convert_checkpoint import unpack_offline_uint8

    rng = np.random.default_rng(7)
    q = rng.integers(-1, 2, size=(64, 32)).astype(np.int8)
    codes = (q + 1).astype(np.uint8).reshape(4, 16, 32)
    packed = codes[0] | (codes[1] << 2) | (codes[2] << 4) | (codes[3] << 6)
    assert np.array_equal(unpack_offline_uint8(torch.from_numpy(packed)).numpy(), q)


def test_hf_name_mapping_and_fusion():
    from bitnet_b200.config import preset
    from bitnet_b200.convert_checkpoint import convert_hf_state_dict, rope_rows_to_interleaved

    args = preset("tiny")
    d, hd = args.dim, args.head_dim
    g = torch.Generator().manual_seed(1)
    st = {"model.embed_tokens.weight": torch.randn(args.vocab_size, d, generator=g), "model.norm.weight": torch.ones(d)}
    for i in range(args.n_layers):
        b = f"model.layers.{i}."
        st[b + "self_attn.q_proj.weight"] = torch.randn(args.n_heads * hd, d, generator=g)
        st[b + "self_attn.k_proj.weight"] = torch.randn(args.n_kv_heads * hd, d, generator=g)
        st[b + "self_attn.v_proj.weight"] = torch.randn(args.n_kv_heads * hd, d, generator=g)
        st[b + "self_attn.o_proj.weight"] = torch.randn(d, d, generator=g)
        st[b + "mlp.gate_proj.weight"] = torch.randn(args.ffn_dim, d, generator=g)
        st[b + "mlp.up_proj.weight"] = torch.randn(args.ffn_dim, d, generator=g)
        st[b + "mlp.down_proj.weight"] = torch.randn(d, args.ffn_dim, generator=g)
        for nm in ("input_layernorm", "post_attention_layernorm", "self_attn.attn_sub_norm"):
            st[b + nm + ".weight"] = torch.ones(d)
        st[b + "mlp.ffn_sub_norm.weight"] = torch.ones(args.ffn_dim)
    out = convert_hf_state_dict(st, args)
    wqkv = out["layers.1.attention.wqkv.weight"]
    assert wqkv.shape == ((args.n_heads + 2 * args.n_kv_heads) * hd, d)
    assert torch.equal(wqkv[: args.n_heads * hd], rope_rows_to_interleaved(st["model.layers.1.self_attn.q_proj.weight"], args.n_heads))
    assert torch.equal(wqkv[-args.n_kv_heads * hd:], st["model.layers.1.self_attn.v_proj.weight"])
    assert torch.equal(out["layers.0.feed_forward.w13.weight"][args.ffn_dim:], st["model.layers.0.mlp.up_proj.weight"])
    assert out["output.weight"] is st["model.embed_tokens.weight"]


# ---------------------------------------------------------------------------- GPU parts


@pytest.mark.gpu
def test_convert_checkpoint_scale_assembly_and_model_equivalence():
    """convert_hf_state_dict + convert_ts_checkpoint + load_int2_state give a model whose
    BitLinears hold exactly np_oracle.ternarize of every sub-matrix, weight_scale =
    [s_q, s_k, s_v, 0] / [s_1, s_3, 0, 0] / [s, 0, 0, 0] (gpu/convert_checkpoint.py:41-83),
    and the reference's own int2 packing of the same weights re-tiles to the same bytes."""
    from bitnet_b200 import pack_weight
    from bitnet_b200.config import preset
    from bitnet_b200.convert_checkpoint import (convert_reference_int2_state, convert_ts_checkpoint, load_int2_state)
    from bitnet_b200.model import Transformer

    args = preset("tiny")
    g = torch.Generator().manual_seed(2)
    d, hd, F = args.dim, args.head_dim, args.ffn_dim
    state = {"tok_embeddings.weight": torch.randn(args.vocab_size, d, generator=g).bfloat16(),
             "norm.weight": torch.ones(d).bfloat16()}
    state["output.weight"] = state["tok_embeddings.weight"]
    for i in range(args.n_layers):
        b = f"layers.{i}."
        state[b + "attention.wqkv.weight"] = torch.randn((args.n_heads + 2 * args.n_kv_heads) * hd, d, generator=g)
        state[b + "attention.wo.weight"] = torch.randn(d, d, generator=g) * 0.3
        state[b + "feed_forward.w13.weight"] = torch.cat([torch.randn(F, d, generator=g) * 2.0, torch.randn(F, d, generator=g) * 0.5])
        state[b + "feed_forward.w2.weight"] = torch.randn(d, F, generator=g)
        for nm, n in (("attention_norm", d), ("ffn_norm", d), ("attention.attn_sub_norm", d), ("feed_forward.ffn_sub_norm", F)):
            state[b + nm + ".weight"] = (1 + 0.1 * torch.randn(n, generator=g)).bfloat16()
    int2, fp16 = convert_ts_checkpoint(state, args, device="cuda", want_fp16=True)
    key = "layers.1.attention.wqkv.weight"
    w = state[key].numpy()
    sizes = [args.n_heads * hd, args.n_kv_heads * hd, args.n_kv_heads * hd]
    qs, ss, lo = [], [], 0
    for n in sizes:
        q, s = O.ternarize(w[lo:lo + n])
        qs.append(q)
        ss.append(O.to_bf16(np.array([s], dtype=np.float32))[0])
        lo += n
    q_all = np.concatenate(qs)
    got_q = pack_weight.unpack_int2_to_int8(int2[key], *w.shape).cpu().numpy()
    assert np.array_equal(got_q, q_all)
    ws = int2[key.replace("weight", "weight_scale")].float().cpu().numpy()
    assert ws.shape == (4,) and np.array_equal(ws[:3], np.array(ss, dtype=np.float32)) and ws[3] == 0
    ws13 = int2["layers.0.feed_forward.w13.weight_scale"].float().cpu().numpy()
    assert ws13[2] == 0 and ws13[3] == 0 and ws13[0] != ws13[1]
    assert np.allclose(fp16[key].numpy(), np.concatenate([q * s for q, s in zip(qs, ss)]), rtol=1e-2)
    # the reference's packing of the same ternary weights converts to the same W2T bytes
    ref_state = {key: torch.from_numpy(O.ref_gpu_pack(q_all))}
    assert torch.equal(convert_reference_int2_state(ref_state)[key], int2[key])
    # and the state loads into the kernel model
    with torch.device("meta"):
        model = Transformer(args, 32)
    model = load_int2_state(model.to_empty(device="cuda"), int2)
    lin = model.layers[1].attention.wqkv
    assert torch.equal(lin.weight, int2[key]) and np.array_equal(lin.scale_f32.cpu().numpy(), np.array(ss, dtype=np.float32))


@pytest.mark.gpu
def test_gguf_round_trip_gives_the_same_logits(tmp_path):
    """write -> read -> bitnet_pack_from_i2s -> logits equal to those of a model whose BitLinears
    were packed from the very same ternary values through bitnet_pack_ternary."""
    from bitnet_b200 import gguf_i2s as G
    from bitnet_b200.model import Transformer, make_cache, rope_table

    path = str(tmp_path / "dummy.gguf")
    G.generate_dummy_model(path, hidden=256, inter=384, layers=2, heads=4, kv_heads=2, vocab=512, seed=11, size="custom")
    a = G.load_gguf_model(path, device="cuda", max_seq_len=64, rope_interleave=False)
    meta, tensors = G.read_gguf(path)
    args = G.model_args_from_gguf(meta)
    with torch.device("meta"):
        b = Transformer(args, 64)
    b = b.to_empty(device="cuda")
    dev = lambda name: torch.from_numpy(np.asarray(tensors[name].data).astype(np.float32)).cuda().bfloat16()
    tern = lambda name: (torch.from_numpy(G.unpack_i2_s(np.asarray(tensors[name].data), *tensors[name].shape)).cuda(),
                         torch.tensor(float(G.i2_s_scale(np.asarray(tensors[name].data), int(np.prod(tensors[name].shape))))))
    b.tok_embeddings.weight.data = dev("token_embd.weight")
    b.output.weight = b.tok_embeddings.weight
    b.norm.weight.data = dev("output_norm.weight")
    for i, layer in enumerate(b.layers):
        p = f"blk.{i}."
        for lin, names in ((layer.attention.wqkv, ["attn_q", "attn_k", "attn_v"]), (layer.attention.wo, ["attn_output"]),
                           (layer.feed_forward.w13, ["ffn_gate", "ffn_up"]), (layer.feed_forward.w2, ["ffn_down"])):
            parts, scales = zip(*(tern(p + n + ".weight") for n in names))
            lin.load_ternary(parts, scales)
        layer.attention_norm.weight.data = dev(p + "attn_norm.weight")
        layer.ffn_norm.weight.data = dev(p + "ffn_norm.weight")
        layer.attention.attn_sub_norm.weight.data = dev(p + "attn_sub_norm.weight")
        layer.feed_forward.ffn_sub_norm.weight.data = dev(p + "ffn_sub_norm.weight")
    b.rope = rope_table(args.head_dim, 64, args.rope_theta, "cuda")
    for la, lb in zip(a.layers, b.layers):
        assert torch.equal(la.attention.wqkv.weight, lb.attention.wqkv.weight)
        assert torch.equal(la.feed_forward.w2.weight, lb.feed_forward.w2.weight)
        assert torch.equal(la.feed_forward.w13.scale_f32, lb.feed_forward.w13.scale_f32)
    toks = torch.randint(0, args.vocab_size, (2, 9), device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    pos = torch.zeros(2, dtype=torch.int64, device="cuda")
    la = a(toks, pos, make_cache(args, 2, 64, "cuda"), kv_len=9)
    lb = b(toks, pos, make_cache(args, 2, 64, "cuda"), kv_len=9)
    assert torch.equal(la, lb)
    # with the rotary row permutation the q rows move inside their heads and nothing else changes
    c = G.load_gguf_model(path, device="cuda", max_seq_len=64, rope_interleave=True)
    assert torch.equal(c.layers[0].attention.wo.weight, a.layers[0].attention.wo.weight)
    assert not torch.equal(c.layers[0].attention.wqkv.weight, a.layers[0].attention.wqkv.weight)
