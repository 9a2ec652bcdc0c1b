"""Generates the files under tests/golden/ (MoE layer, weight rounding, Hunyuan3D MoE, attention, blocks, whole model)
by running the UNMODIFIED reference.

Usage (in a container that has the reference tree; it is not needed at test time):

    python tests/golden/make_golden.py /path/to/ComfyUI

The script imports the reference's ``comfy.ldm.hidream.model.MOEFeedForwardSwiGLU`` and ``comfy.ops`` on
the CPU, loads seeded synthetic weights through ``load_state_dict(strict=True)`` (which also pins the
state-dict key set), runs ``MoEGate.forward``, ``MOEFeedForwardSwiGLU.forward`` and ``moe_infer`` and stores
the results.  bf16 tensors are stored up-cast to fp32 (exact).
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import hidream_moe_oracle as O  # noqa: E402  (seeded weight recipe only)
from oracle import hunyuan3d_moe_oracle as H  # noqa: E402  (seeded weight recipe only)
from oracle import hidream_attention_oracle as A  # noqa: E402  (seeded weight recipe only)
from oracle import hidream_block_oracle as B  # noqa: E402  (seeded weight recipe only)

DIM, HIDDEN_DIM, E, K = 256, 1024, 4, 2
BATCH, SEQ = 2, 64
W_SEED, X_SEED = 0, 1


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from comfy.cli_args import args
    args.cpu = True
    import comfy.model_management  # noqa: F401
    import comfy.ops
    from comfy.ldm.hidream.model import MOEFeedForwardSwiGLU

    torch.manual_seed(0)
    out = {}
    meta = dict(dim=DIM, hidden_dim=HIDDEN_DIM, n_experts=E, top_k=K, batch=BATCH, seq=SEQ, w_seed=W_SEED,
                x_seed=X_SEED, torch_version=torch.__version__)

    def build(ops, dtype, layer):
        m = MOEFeedForwardSwiGLU(DIM, HIDDEN_DIM, E, K, dtype=dtype, device="cpu", operations=ops)
        missing = m.load_state_dict(layer, strict=True)
        assert not missing.missing_keys and not missing.unexpected_keys
        return m.eval()

    def f32(t):
        return t.detach().float().numpy()

    def run_case(name, m, x, gate_in_fp32):
        n = BATCH * SEQ
        with torch.no_grad():
            if gate_in_fp32:
                idx, w, _ = m.gate(x.float())
                w = w.to(x.dtype)
            else:
                idx, w, _ = m.gate(x)
            x2 = x.view(n, DIM)
            routed = m.moe_infer(x2, idx.view(-1), w.view(-1, 1))
            shared = m.shared_experts(x2)
            full = routed + shared
            out[f"{name}/idx"] = idx.numpy().astype(np.int64)
            out[f"{name}/w"] = f32(w)
            out[f"{name}/routed"] = f32(routed)
            out[f"{name}/shared"] = f32(shared)
            out[f"{name}/out"] = f32(full)
            if not gate_in_fp32:
                fwd = m.forward(x.clone())
                out[f"{name}/forward"] = f32(fwd.view(n, DIM))
                # both branches of the reference agree bit for bit when fed the same routing
                meta[f"{name}_forward_equals_infer"] = bool(torch.equal(fwd.view(n, DIM), full))

    x32 = O.make_input(BATCH * SEQ, DIM, X_SEED).view(BATCH, SEQ, DIM)
    layer32 = O.make_layer(DIM, HIDDEN_DIM, E, W_SEED)
    out["x_checksum"] = np.array([float(x32.double().sum()), float(x32.double().abs().sum())])
    out["w_checksum"] = np.array([float(sum(v.double().sum() for v in layer32.values())),
                                  float(sum(v.double().abs().sum() for v in layer32.values()))])

    # fp32, as shipped (configuration 1 of the benchmark spec, reduced size)
    m = build(comfy.ops.disable_weight_init, torch.float32, layer32)
    run_case("fp32", m, x32, gate_in_fp32=False)

    # bf16 as shipped (gate in bf16) and with the fp32 gate of the parity contract
    xb = x32.bfloat16()
    layer16 = {k: v.bfloat16() for k, v in layer32.items()}
    m = build(comfy.ops.disable_weight_init, torch.bfloat16, layer16)
    run_case("bf16_shipped", m, xb, gate_in_fp32=False)
    run_case("bf16", m, xb, gate_in_fp32=True)

    # feed-forward half of a block exactly as HiDreamImageSingleTransformerBlock.forward spells it
    # (comfy/ldm/hidream/model.py:429-433), with the reference's LayerNorm op and the bf16 module built above
    norm3 = comfy.ops.disable_weight_init.LayerNorm(DIM, eps=1e-06, elementwise_affine=False)
    shift_mlp, scale_mlp, gate_mlp = O.make_modulation(BATCH, DIM)
    with torch.no_grad():
        image_tokens = xb
        wtype = image_tokens.dtype
        norm_image_tokens = norm3(image_tokens).to(dtype=wtype)
        norm_image_tokens = norm_image_tokens * (1 + scale_mlp) + shift_mlp
        ff_output_i = gate_mlp * m(norm_image_tokens.to(dtype=wtype))
        out["block_bf16/normed"] = f32(norm_image_tokens.reshape(-1, DIM))
        out["block_bf16/out"] = f32((ff_output_i + image_tokens).reshape(-1, DIM))
        dense = gate_mlp * m.shared_experts(norm_image_tokens) + image_tokens
        out["block_bf16/dense_out"] = f32(dense.reshape(-1, DIM))

    # scaled fp8 weights, three flavours of comfy.ops.scaled_fp8_ops
    layer8 = O.quantize_layer_fp8(layer16)
    ops = comfy.ops.scaled_fp8_ops(fp8_matrix_mult=False, scale_input=False, override_dtype=torch.float8_e4m3fn)
    m = build(ops, torch.bfloat16, layer8)
    run_case("fp8_dequant", m, xb, gate_in_fp32=True)

    ops = comfy.ops.scaled_fp8_ops(fp8_matrix_mult=True, scale_input=False, override_dtype=torch.float8_e4m3fn)
    m = build(ops, torch.bfloat16, layer8)
    run_case("fp8_matmul", m, xb, gate_in_fp32=True)

    layer8s = O.quantize_layer_fp8(layer16, scale_input=0.75)
    ops = comfy.ops.scaled_fp8_ops(fp8_matrix_mult=True, scale_input=True, override_dtype=torch.float8_e4m3fn)
    m = build(ops, torch.bfloat16, layer8s)
    run_case("fp8_matmul_scale_input", m, xb, gate_in_fp32=True)

    out["state_dict_keys"] = np.array(sorted(layer8s.keys()))
    out["meta_keys"] = np.array(sorted(meta.keys()))
    out["meta_vals"] = np.array([str(meta[k]) for k in sorted(meta.keys())])
    path = os.path.join(HERE, "hidream_moe_small.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")
    for k in sorted(meta):
        print(" ", k, meta[k])


def hunyuan3d(ref_root: str) -> None:
    """MoEBlock of comfy/ldm/hunyuan3dv2_1/hunyuandit.py at reduced size: 8 experts, top-2, GELU feed-forwards."""
    import comfy.ops
    from comfy.ldm.hunyuan3dv2_1.hunyuandit import MoEBlock

    dim, inner, n_exp, k, batch, seq = 256, 1024, 8, 2, 2, 64
    n = batch * seq
    out = {}

    def f32(t):
        return t.detach().float().numpy()

    x32 = H.make_input(n, dim, X_SEED).view(batch, seq, dim)
    for name, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        layer = H.make_layer(dim, inner, n_exp, W_SEED, dtype=dtype)
        m = MoEBlock(dim, num_experts=n_exp, moe_top_k=k, ff_inner_dim=inner, operations=comfy.ops.disable_weight_init,
                     device="cpu", dtype=dtype)
        res = m.load_state_dict(layer, strict=True)
        assert not res.missing_keys and not res.unexpected_keys
        x = x32.to(dtype)
        with torch.no_grad():
            m.eval()
            out[f"{name}/forward"] = f32(m(x.clone()).view(n, dim))            # as shipped: gate in x.dtype
            idx_s, w_s, _ = m.gate(x)
            out[f"{name}/idx_shipped"] = idx_s.numpy().astype(np.int64)
            out[f"{name}/w_shipped"] = f32(w_s)
            idx, w, _ = m.gate(x.float())                                         # the parity contract's fp32 gate
            w = w.to(dtype)
            x2 = x.view(n, dim)
            routed = m.moe_infer(x2, idx.view(-1), w.view(-1, 1))
            shared = m.shared_experts(x2)
            out[f"{name}/idx"] = idx.numpy().astype(np.int64)
            out[f"{name}/w"] = f32(w)
            out[f"{name}/routed"] = f32(routed)
            out[f"{name}/shared"] = f32(shared)
            out[f"{name}/out"] = f32(routed + shared)
            m.train()
            out[f"{name}/forward_train_branch"] = f32(m(x.clone()).view(n, dim))
    out["state_dict_keys"] = np.array(sorted(layer.keys()))
    out["meta_keys"] = np.array(["dim", "inner", "n_experts", "top_k", "batch", "seq", "w_seed", "x_seed", "torch_version"])
    out["meta_vals"] = np.array([str(v) for v in (dim, inner, n_exp, k, batch, seq, W_SEED, X_SEED, torch.__version__)])
    path = os.path.join(HERE, "hunyuan3d_moe_small.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def attention(ref_root: str) -> None:
    """HiDreamAttention with HiDreamAttnProcessor_flashattn (comfy/ldm/hidream/model.py:79-213) at reduced size, as a
    double-stream (image + text) and as a single-stream block; q, k, v are captured where the processor hands them to
    the attention call."""
    import comfy.ldm.hidream.model as RM
    import comfy.ops

    heads, head_dim, axes = 4, 64, [32, 16, 16]
    dim = heads * head_dim
    batch, hh, ww, n_text = 2, 6, 8, 16
    out = {}
    captured = {}
    stock = RM.attention

    def spy(query, key, value, transformer_options={}):
        captured.update(q=query.clone(), k=key.clone(), v=value.clone())
        return stock(query, key, value, transformer_options=transformer_options)

    RM.attention = spy
    # On a CUDA device the reference selects attention_pytorch (comfy/ldm/modules/attention.py:634-635); with --cpu it
    # would pick the sub-quadratic variant.  The fixtures pin the function a B200 runs.
    import comfy.ldm.modules.attention as RA

    stock_select = RM.optimized_attention
    RM.optimized_attention = RA.attention_pytorch

    def f32(t):
        return t.detach().float().numpy()

    ids = A.make_ids(batch, hh, ww, n_text)
    freqs = RM.EmbedND(theta=10000, axes_dim=axes)(ids)
    out["rope"] = f32(freqs)
    g = torch.Generator().manual_seed(X_SEED)
    img32 = torch.randn((batch, hh * ww, dim), generator=g)
    txt32 = torch.randn((batch, n_text, dim), generator=g)
    out["x_checksum"] = np.array([float(img32.double().sum()), float(txt32.double().sum())])
    for name, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        for single in (False, True):
            tag = f"{name}/{'single' if single else 'double'}"
            layer = A.make_layer(dim, heads, head_dim, single, seed=W_SEED, dtype=dtype)
            m = RM.HiDreamAttention(query_dim=dim, heads=heads, dim_head=head_dim,
                                    processor=RM.HiDreamAttnProcessor_flashattn(), single=single, dtype=dtype,
                                    device="cpu", operations=comfy.ops.disable_weight_init)
            res = m.load_state_dict(layer, strict=True)
            assert not res.missing_keys and not res.unexpected_keys
            img, txt = img32.to(dtype), txt32.to(dtype)
            with torch.no_grad():
                if single:
                    # a single-stream block attends over the concatenated sequence with the image projections
                    seq = torch.cat([img, txt], dim=1)
                    y = m(seq, None, None, rope=freqs)
                    out[f"{tag}/out"] = f32(y)
                else:
                    yi, yt = m(img, None, txt, rope=freqs)
                    out[f"{tag}/out_i"], out[f"{tag}/out_t"] = f32(yi), f32(yt)
            for k in ("q", "k", "v"):
                out[f"{tag}/{k}"] = f32(captured[k])
            out[f"{tag}/keys"] = np.array(sorted(layer.keys()))
    RM.attention = stock
    RM.optimized_attention = stock_select
    out["meta_keys"] = np.array(["heads", "head_dim", "axes", "batch", "height", "width", "n_text", "w_seed", "x_seed",
                                 "torch_version"])
    out["meta_vals"] = np.array([str(v) for v in (heads, head_dim, axes, batch, hh, ww, n_text, W_SEED, X_SEED,
                                                  torch.__version__)])
    path = os.path.join(HERE, "hidream_attention_small.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def blocks(ref_root: str) -> None:
    """HiDreamImageTransformerBlock and HiDreamImageSingleTransformerBlock (comfy/ldm/hidream/model.py:363-524) at
    reduced size, as shipped (MoE gate in the activation dtype), with the attention variant a CUDA device selects."""
    import comfy.ldm.hidream.model as RM
    import comfy.ldm.modules.attention as RA
    import comfy.ops

    heads, head_dim, axes, n_exp = 4, 64, [32, 16, 16], 4
    dim = heads * head_dim
    batch, hh, ww, n_text = 2, 6, 8, 16
    stock_select = RM.optimized_attention
    RM.optimized_attention = RA.attention_pytorch
    out = {}

    def f32(t):
        return t.detach().float().numpy()

    freqs = RM.EmbedND(theta=10000, axes_dim=axes)(A.make_ids(batch, hh, ww, n_text))
    g = torch.Generator().manual_seed(X_SEED)
    img32 = torch.randn((batch, hh * ww, dim), generator=g)
    txt32 = torch.randn((batch, n_text, dim), generator=g)
    ada32 = torch.randn((batch, dim), generator=g)
    for name, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        img, txt, ada = img32.to(dtype), txt32.to(dtype), ada32.to(dtype)
        for single in (False, True):
            cls = RM.HiDreamImageSingleTransformerBlock if single else RM.HiDreamImageTransformerBlock
            layer = B.make_layer(dim, heads, head_dim, n_exp, single, seed=W_SEED, dtype=dtype)
            m = cls(dim, heads, head_dim, n_exp, 2, dtype=dtype, device="cpu", operations=comfy.ops.disable_weight_init)
            res = m.load_state_dict(layer, strict=True)
            assert not res.missing_keys and not res.unexpected_keys
            tag = f"{name}/{'single' if single else 'double'}"
            with torch.no_grad():
                if single:
                    out[f"{tag}/out"] = f32(m(torch.cat([img, txt], dim=1), None, None, ada, freqs))
                else:
                    yi, yt = m(img, None, txt, ada, freqs)
                    out[f"{tag}/out_i"], out[f"{tag}/out_t"] = f32(yi), f32(yt)
            out[f"{tag}/keys"] = np.array(sorted(layer.keys()))
    RM.optimized_attention = stock_select
    out["meta_keys"] = np.array(["heads", "head_dim", "axes", "n_experts", "batch", "height", "width", "n_text",
                                 "w_seed", "x_seed", "torch_version"])
    out["meta_vals"] = np.array([str(v) for v in (heads, head_dim, axes, n_exp, batch, hh, ww, n_text, W_SEED, X_SEED,
                                                  torch.__version__)])
    path = os.path.join(HERE, "hidream_block_small.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def model(ref_root: str) -> None:
    """HiDreamImageTransformer2DModel (comfy/ldm/hidream/model.py:571-829) at reduced depth and width, one denoising
    step: as shipped in fp32 and bf16, and in bf16 with the MoE gates evaluated on the fp32 copy of their input (the
    routing convention the kernels follow: indices from the fp32 gate, weights cast back to the activation dtype).
    The attention variant is the one a CUDA device selects."""
    import comfy.ldm.hidream.model as RM
    import comfy.ldm.modules.attention as RA
    import comfy.ops

    from oracle import hidream_model_recipe as R

    stock_select, stock_gate = RM.optimized_attention, RM.MoEGate.forward
    RM.optimized_attention = RA.attention_pytorch

    def gate_on_fp32_copy(self, hidden_states):
        # the reference's own MoEGate.forward, handed x.float(): nothing inside the module is changed
        idx, w, aux = stock_gate(self, hidden_states.float())
        return idx, w.to(hidden_states.dtype), aux

    out = {}
    keys = None
    for name, dtype, fp32_gate in (("fp32", torch.float32, False), ("bf16", torch.bfloat16, False),
                                   ("bf16_fp32gate", torch.bfloat16, True)):
        m = RM.HiDreamImageTransformer2DModel(**R.CONFIG, dtype=dtype, device="cpu",
                                              operations=comfy.ops.disable_weight_init).eval()
        shapes = {k: v.shape for k, v in m.state_dict().items()}
        res = m.load_state_dict(R.make_state(shapes, dtype), strict=True)
        assert not res.missing_keys and not res.unexpected_keys
        keys = list(shapes.keys())
        RM.MoEGate.forward = gate_on_fp32_copy if fp32_gate else stock_gate
        with torch.no_grad():
            out[f"{name}/out"] = m(*R.make_inputs(dtype)).detach().float().numpy()
    RM.MoEGate.forward = stock_gate
    RM.optimized_attention = stock_select
    out["keys"] = np.array(keys)
    out["shapes"] = np.array([",".join(str(d) for d in shapes[k]) for k in keys])
    out["torch_version"] = np.array([torch.__version__])
    path = os.path.join(HERE, "hidream_model_small.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def rounding_input(dtype):
    """Seeded tensor with the edge cases of the stochastic rounding in its first row."""
    g = torch.Generator().manual_seed(11)
    v = (torch.randn((96, 160), generator=g) * 3).to(dtype)
    edge = [0.0, -0.0, 448.0, 500.0, -1000.0, 2.0 ** -9, 2.0 ** -10, 1.999, 0.9995, 255.9, -0.0625, 3.0e-3, 7.0e4,
            float("inf"), -float("inf"), 15.99]
    v[0, :len(edge)] = torch.tensor(edge).to(dtype)
    return v


def weight_rounding(ref_root: str) -> None:
    """comfy.float.stochastic_rounding (comfy/float.py:50-67) and scaled_fp8_ops.Linear.set_weight
    (comfy/ops.py:418-426) on seeded tensors with the CPU generator."""
    import comfy.float
    import comfy.ops

    out = {}
    for name, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        v = rounding_input(dtype)
        for tname, target in (("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
            for seed in (0, 7):
                q = comfy.float.stochastic_rounding(v.clone(), target, seed=seed)
                out[f"{name}/{tname}/seed{seed}"] = q.view(torch.uint8).numpy()
    ops = comfy.ops.scaled_fp8_ops(fp8_matrix_mult=True, scale_input=False, override_dtype=torch.float8_e4m3fn)
    lin = ops.Linear(160, 96, bias=False, dtype=torch.bfloat16, device="cpu")
    lin.scale_weight.data.fill_(0.0123)
    lin.set_weight(rounding_input(torch.float32), seed=3)
    out["set_weight/seed3"] = lin.weight.data.view(torch.uint8).numpy()
    out["torch_version"] = np.array([torch.__version__])
    path = os.path.join(HERE, "weight_rounding.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def _import_reference(ref_root: str) -> None:
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    from comfy.cli_args import args
    args.cpu = True
    import comfy.model_management  # noqa: F401


if __name__ == "__main__":
    # python tests/golden/make_golden.py ROOT [part ...]    parts: moe rounding hunyuan3d attention blocks model
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("COMFYUI_ROOT", "ComfyUI")
    parts = sys.argv[2:] or ["moe", "rounding", "hunyuan3d", "attention", "blocks", "model"]
    _import_reference(root)
    table = {"moe": main, "rounding": weight_rounding, "hunyuan3d": hunyuan3d, "attention": attention,
             "blocks": blocks, "model": model}
    for part in parts:
        table[part](root)
