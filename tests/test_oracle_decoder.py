"""The NumPy decoder of oracle/ref_decoder.py against the plain-PyTorch fake-quantised form of
the same model (bitnet_b200.model with use_kernel=False), both on the CPU: two independent
statements of gpu/model.py's decode step must agree."""
import numpy as np
import torch

from oracle import np_oracle as O
from oracle.ref_decoder import OracleDecoder, OracleLinear


def test_oracle_decoder_matches_pytorch_fake_quant_model(port_lib):
    from bitnet_b200.model import build_synthetic, make_cache, preset

    args = preset("tiny", use_kernel=False)
    max_seq = 32
    model = build_synthetic(args, seed=9, device="cpu", max_seq_len=max_seq)
    dec = OracleDecoder(args.dim, args.n_heads, args.n_kv_heads, args.ffn_dim, args.vocab_size, args.norm_eps,
                        args.rope_theta, max_seq, gemm_lib=port_lib)
    f = lambda t: t.detach().float().numpy()
    dec.set_rope(f(model.rope[:max_seq]))
    dec.emb, dec.out_w, dec.final_norm = f(model.tok_embeddings.weight), f(model.output.weight), f(model.norm.weight)
    for layer in model.layers:
        att, ff = layer.attention, layer.feed_forward

        def lin(m):
            scales, ends, lo = [], [], 0
            for n in m._segments:
                scales.append(float(m.row_scale[lo]))
                lo += n
                ends.append(lo)
            return OracleLinear.from_ternary(m.ternary.numpy().astype(np.int8), scales, ends)

        dec.add_layer(lin(att.wqkv), lin(att.wo), lin(ff.w13), lin(ff.w2), f(layer.attention_norm.weight),
                      f(att.attn_sub_norm.weight), f(layer.ffn_norm.weight), f(ff.ffn_sub_norm.weight))
    B = 2
    dec.reset(B)
    cache = make_cache(args, B, max_seq, device="cpu")
    rng = np.random.default_rng(3)
    errs = []
    for step in range(10):
        tok = rng.integers(0, args.vocab_size, size=B)
        pos = torch.full((B,), step, dtype=torch.int64)
        # layer by layer on the same input: the quantisers amplify last-bit differences, which a
        # 256-wide random model then carries from layer to layer
        h = model.tok_embeddings(torch.from_numpy(tok)[:, None])
        for li, (layer, c) in enumerate(zip(model.layers, cache)):
            want = layer(h, c, pos, model.rope)
            got = dec.layer_forward(li, f(h)[:, 0], pos.numpy())
            w = f(want)[:, 0]
            errs.extend((np.abs(got - w).max(-1) / np.abs(w).max(-1)).tolist())
            h = want
        want = f(model.output(model.norm(h)))[:, 0]
        got = dec.head(f(h)[:, 0])
        errs.extend((np.abs(got - want).max(-1) / np.abs(want).max(-1)).tolist())
    # PyTorch runs its attention in bf16; a 256-wide model turns one flipped int8 value into ~1 %
    assert np.median(errs) <= 1e-2 and max(errs) <= 5e-2, (np.median(errs), max(errs))
