"""Generate the golden fixtures under tests/golden/ by RUNNING THE REFERENCE on CPU.

Usage (only where the reference checkout is available; the fixtures are committed so
the test-suite itself never needs it):

    PYTHONPATH=<reference root> python tests/golden/make_golden.py

For each case the reference's own code does all of the work:
  * CMSBlockLinear.prune_step_blocks / carve            (topology + BCSR metadata)
  * deploy_quant.pack_mortar_ternary / unpack_ternary   (codes, scale, flat 2-bit pack)
  * fused_decode_step.mortar_pack_strips                (decode strip layout + work list)
  * engine._mortar_dense                                (dense reconstruction)
  * routing.TileRouter.forward                          (gates)
  * transformer._SwiGLUMortar.forward in dense mode on the reconstructed weights
    (fp32, and bf16 under CPU autocast = the prefill rounding points)
  * attention.RMSNorm                                   (decode prologue)
The carved forward itself (morph_stk::dds) is CUDA/Triton-only in the reference, so the
dense-reconstruction forward is the reference's CPU path for this MLP.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16)


def build_case(name, d_model, d_ff, blocking, n_clusters, ratio, x_shape, seed, density=0.25):
    from morph.model.transformer import _SwiGLUMortar
    from morph.model.attention import RMSNorm
    from morph.inference.deploy_quant import pack_mortar_ternary, unpack_ternary
    from morph.inference.engine import _mortar_dense
    from morph.kernels.triton.fused_decode_step import mortar_pack_strips

    out = {}
    torch.manual_seed(seed)
    mlp = _SwiGLUMortar(d_model, d_ff)
    w_gu = (torch.randn(2 * d_ff, d_model) * 0.02).to(torch.bfloat16).float()
    w_dn = (torch.randn(d_model, d_ff) * 0.02).to(torch.bfloat16).float()
    out["w_gu_bf16"] = _bf16_bits(w_gu)
    out["w_dn_bf16"] = _bf16_bits(w_dn)
    dense_w = {}
    for tag, lin, w in (("gu", mlp.gate_up, w_gu), ("dn", mlp.down, w_dn)):
        cms = lin._cms
        with torch.no_grad():
            cms.weight.copy_(w)
            t = cms.tile_size
            tiles = w.reshape(cms.R, t, cms.C, t)
            cms.block_score_ema.copy_(tiles.pow(2).sum(dim=(1, 3)).sqrt())
        out[f"{tag}_tile_scores"] = cms.block_score_ema.numpy().copy()
        cms.prune_step_blocks(prune_rate=1.0 - density, target_density=density,
                              blocking=blocking)
        out[f"{tag}_prune_mask"] = cms._prune_mask.numpy().copy()
        nnz = cms.carve(blocking=blocking)
        out[f"{tag}_data_bf16"] = _bf16_bits(cms.mortar_data.data)
        for k in ("row_indices", "column_indices", "offsets", "column_indices_t",
                  "offsets_t", "block_offsets_t"):
            out[f"{tag}_{k}"] = getattr(cms, f"mortar_{k}").numpy().copy()
        info = pack_mortar_ternary(cms)
        out[f"{tag}_packed"] = cms.mortar_packed.numpy().copy()
        out[f"{tag}_scale"] = np.float32(cms.mortar_scale.item())
        out[f"{tag}_nonzero_frac"] = np.float64(info["nonzero_code_frac"])
        codes = unpack_ternary(cms.mortar_packed, cms._packed_numel, torch.float32)
        out[f"{tag}_codes"] = codes.view(nnz, blocking, blocking).to(torch.int8).numpy()
        strips, col_idx, offsets, scale, O, ent, nspl_max, cnts = mortar_pack_strips(cms)
        out[f"{tag}_strips"] = strips.numpy()
        out[f"{tag}_ent"] = ent.numpy()
        out[f"{tag}_cnts"] = cnts.numpy()
        out[f"{tag}_nspl_max"] = np.int32(nspl_max)
        dense_w[tag] = _mortar_dense(cms)
        out[f"{tag}_dense_checksum"] = np.float64(dense_w[tag].double().abs().sum().item())

    # Dense twin that carries the reconstructed effective weights: the reference's CPU
    # path for the carved MLP.
    torch.manual_seed(seed + 1)
    twin = _SwiGLUMortar(d_model, d_ff)
    with torch.no_grad():
        twin.gate_up._cms.weight.copy_(dense_w["gu"])
        twin.down._cms.weight.copy_(dense_w["dn"])
    twin.eval()
    x = torch.randn(*x_shape, d_model)
    norm = RMSNorm(d_model)
    with torch.no_grad():
        norm.weight.copy_(1.0 + 0.1 * torch.randn(d_model))
    out["x_raw"] = x.numpy().copy()
    out["rms_weight"] = norm.weight.detach().numpy().copy()
    with torch.no_grad():
        xn = norm(x)
    out["x_normed"] = xn.numpy().copy()
    xb = xn.to(torch.bfloat16).float()          # bf16-representable activations
    out["x_bf16"] = _bf16_bits(xb)

    with torch.no_grad():
        out["y_fp32"] = twin(xb).numpy().copy()
        with torch.autocast("cpu", dtype=torch.bfloat16):
            yb = twin(xb)
        assert yb.dtype == torch.bfloat16
        out["y_bf16"] = _bf16_bits(yb)

    # Routed: attach the reference router, record the gates it emits, and the gated output.
    torch.manual_seed(seed + 2)
    twin.enable_routing(n_clusters=n_clusters, activation_ratio=ratio, n_iters=2)
    with torch.no_grad():
        twin.router.group_bias.copy_(0.5 * torch.randn(n_clusters))
        twin.router.iter_embed.copy_(0.1 * torch.randn_like(twin.router.iter_embed))
    got = {}
    twin.router.register_forward_hook(lambda m, i, o: got.__setitem__("gates", o[0].detach()))
    with torch.no_grad():
        y_r = twin(xb, iter_idx=1)
        out["gates_fp32"] = got["gates"].float().numpy().copy()
        out["y_routed_fp32"] = y_r.numpy().copy()
        with torch.autocast("cpu", dtype=torch.bfloat16):
            y_rb = twin(xb, iter_idx=1)
        out["gates_autocast"] = got["gates"].float().numpy().copy()
        out["y_routed_bf16"] = _bf16_bits(y_rb)
    out["k"] = np.int32(twin.router.activation_k)
    out["meta"] = np.array([d_model, d_ff, blocking, n_clusters], dtype=np.int32)

    # Raw logits -> gates pairs for the gate formula alone.
    torch.manual_seed(seed + 3)
    from morph.model.routing import TileRouter
    r2 = TileRouter(n_tile_groups=n_clusters, d_model=d_model, activation_ratio=ratio)
    r2.eval()
    cap = {}
    orig_topk = torch.Tensor.topk

    def spy_topk(self, *a, **kw):
        cap.setdefault("logits", self.detach().clone())
        return orig_topk(self, *a, **kw)

    torch.Tensor.topk = spy_topk
    try:
        with torch.no_grad():
            g2, _ = r2(xb.reshape(-1, d_model))
    finally:
        torch.Tensor.topk = orig_topk
    if "logits" in cap and cap["logits"].shape[-1] == n_clusters:
        out["router_logits"] = cap["logits"].numpy().copy()
        out["router_gates"] = g2.numpy().copy()
        # the router's own parameters, so a mirror can be loaded and run on the same input
        for k, v in r2.state_dict().items():
            out["router_sd__" + k.replace(".", "__")] = v.detach().numpy().copy()

    path = os.path.join(HERE, f"{name}.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


def decode_sides():
    """The two steps beside the MLP in the decode engine: the hyper-connection POST write
    (hc_post_reference, the eager twin of _hc_post_fwd_kernel) and a stack of per-layer ternary
    projections packed with the reference's ternary_pack for ternary_gemv_rs (the dense
    product of the dequantised stack is the reference's eager result)."""
    from morph.kernels.triton.fused_hyper_connection import hc_post_reference
    from morph.kernels.triton.fused_decode_step import ternary_pack
    out = {}
    torch.manual_seed(11)
    B, S, n, C = 3, 1, 4, 256
    hres = torch.randn(B, S, n, n) * 0.5
    hpost = torch.rand(B, S, n)
    h = torch.randn(B, S, n, C)
    y = torch.randn(B, S, C) * 0.1
    term = torch.randn(B, S, C) * 0.05
    out["hc_hres"], out["hc_hpost_row"], out["hc_h"] = hres.numpy(), hpost.numpy(), h.numpy()
    out["hc_y"], out["hc_term"] = y.numpy(), term.numpy()
    out["hc_out"] = hc_post_reference(hres, hpost, h, y, None).numpy()
    out["hc_out_term"] = hc_post_reference(hres, hpost, h, y, term).numpy()
    # three ternary layers [48, 128] with their own scales, stacked to one [144, 128] GEMV
    I, O = 128, 48
    packs, scales, dense = [], [], []
    for layer in range(3):
        gamma = 0.01 * (layer + 1)
        w = torch.randint(-1, 2, (O, I)).float() * gamma
        codes, sc = ternary_pack(w)
        packs.append(codes)
        scales.append(sc.reshape(1).expand(O).clone())
        dense.append(w)
    x = torch.randn(5, I)
    out["rs_codes"] = torch.cat(packs).numpy()
    out["rs_row_scale"] = torch.cat(scales).numpy()
    out["rs_x"] = x.numpy()
    out["rs_out"] = torch.nn.functional.linear(x, torch.cat(dense)).numpy()
    path = os.path.join(HERE, "decode_sides.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}")


def known_answers():
    """Tiny known-answer vectors taken from running the reference primitives."""
    from morph.inference.deploy_quant import pack_ternary_codes, unpack_ternary, _ternary_quantize
    out = {}
    q = torch.tensor([-1, 0, 1, 1, 0, -1], dtype=torch.int8)
    p = pack_ternary_codes(q)
    out["pack_in"] = q.numpy()
    out["pack_out"] = p.numpy()
    out["unpack_out"] = unpack_ternary(p, 6, torch.float32).numpy()
    torch.manual_seed(7)
    w = torch.randn(5, 16, 16) * 0.02
    w[0, 0, 0] = 0.0
    qq, sc = _ternary_quantize(w)
    out["tq_w"] = w.numpy()
    out["tq_codes"] = qq.numpy()
    out["tq_scale"] = np.float32(sc.item())
    path = os.path.join(HERE, "known_answers.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}")


def main():
    try:
        import morph  # noqa: F401
    except ImportError:
        sys.exit("put the reference checkout on PYTHONPATH to regenerate the fixtures")
    torch.set_num_threads(1)
    known_answers()
    decode_sides()
    build_case("mlp_tile16_d64", d_model=64, d_ff=128, blocking=16, n_clusters=8, ratio=0.5,
               x_shape=(2, 5), seed=11)
    build_case("mlp_tile16_d128_cs16", d_model=128, d_ff=256, blocking=16, n_clusters=16,
               ratio=0.25, x_shape=(3, 4), seed=23)
    build_case("mlp_blk128_d256", d_model=256, d_ff=512, blocking=128, n_clusters=4, ratio=0.5,
               x_shape=(1, 7), seed=37, density=0.5)


if __name__ == "__main__":
    main()
