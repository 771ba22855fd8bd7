"""Pins the CPU oracle against fixtures produced by running the reference itself
(tests/golden/make_golden.py).  No GPU, no reference checkout needed."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES, bf16_from_bits, load_golden
from oracle import mortar_oracle as orc


def test_known_answer_pack():
    ka = load_golden("known_answers")
    assert orc.pack_ternary_codes(np.array([-1, 0, 1, 1]))[0] == 164      # 0b10100100
    np.testing.assert_array_equal(orc.pack_ternary_codes(ka["pack_in"]), ka["pack_out"])
    np.testing.assert_array_equal(orc.unpack_ternary(ka["pack_out"], 6), ka["unpack_out"].astype(np.int8))


def test_known_answer_quantize():
    ka = load_golden("known_answers")
    q, s = orc.ternary_quantize(torch.from_numpy(ka["tq_w"]))
    np.testing.assert_array_equal(q.numpy(), ka["tq_codes"])
    assert np.float32(s.item()) == ka["tq_scale"]


def test_magic_dequant_all_bytes():
    # the property the reference's proof script pins: decode == stored-1 for every byte/stride
    for byte in range(256):
        for st in range(4):
            assert orc.magic_dequant(byte, st) == float(((byte >> (2 * st)) & 3) - 1)


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_topology_and_carve(case):
    g = load_golden(case)
    d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])
    density = 0.5 if "blk128" in case else 0.25
    for tag, bits in (("gu", g["w_gu_bf16"]), ("dn", g["w_dn_bf16"])):
        w = bf16_from_bits(bits).float()
        scores = orc.tile_l2_scores(w)
        np.testing.assert_allclose(scores.numpy(), g[f"{tag}_tile_scores"], rtol=1e-6)
        mask = orc.prune_blocks_once(torch.from_numpy(g[f"{tag}_tile_scores"]), 1.0 - density,
                                     density, blocking=blk)
        np.testing.assert_array_equal(mask.numpy(), g[f"{tag}_prune_mask"])
        cv = orc.carve(w, mask, blk)
        for k in ("row_indices", "column_indices", "offsets", "offsets_t"):
            np.testing.assert_array_equal(getattr(cv, k).numpy(), g[f"{tag}_{k}"])
        # order inside a column of the transposed arrays is unspecified (unstable argsort):
        # compare as sets per column.
        ot = g[f"{tag}_offsets_t"]
        for c in range(len(ot) - 1):
            a = sorted(cv.block_offsets_t[ot[c]:ot[c + 1]].tolist())
            b = sorted(g[f"{tag}_block_offsets_t"][ot[c]:ot[c + 1]].tolist())
            assert a == b
        np.testing.assert_array_equal(
            cv.data.to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16),
            g[f"{tag}_data_bf16"])
        q, s = orc.ternary_quantize(cv.data)
        np.testing.assert_array_equal(q.numpy(), g[f"{tag}_codes"])
        assert np.float32(s.item()) == g[f"{tag}_scale"]
        np.testing.assert_array_equal(orc.pack_ternary_codes(q.numpy()), g[f"{tag}_packed"])
        np.testing.assert_array_equal(orc.unpack_ternary(g[f"{tag}_packed"], q.numel()),
                                      g[f"{tag}_codes"].reshape(-1))
        W = orc.mortar_dense(q, s, cv.row_indices, cv.column_indices, *w.shape)
        assert abs(W.double().abs().sum().item() - float(g[f"{tag}_dense_checksum"])) < 1e-9


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_strip_pack(case):
    g = load_golden(case)
    for tag in ("gu", "dn"):
        sp = orc.pack_strips(g[f"{tag}_codes"], g[f"{tag}_column_indices"], g[f"{tag}_offsets"],
                             g[f"{tag}_scale"])
        np.testing.assert_array_equal(sp.strips, g[f"{tag}_strips"])
        np.testing.assert_array_equal(sp.ent, g[f"{tag}_ent"])
        np.testing.assert_array_equal(sp.cnts, g[f"{tag}_cnts"])
        assert sp.nspl_max == int(g[f"{tag}_nspl_max"])


def _weights(g):
    d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])
    W = {}
    for tag, (O, I) in (("gu", (2 * d_ff, d_model)), ("dn", (d_model, d_ff))):
        W[tag] = orc.mortar_dense(torch.from_numpy(g[f"{tag}_codes"]),
                                  torch.tensor(g[f"{tag}_scale"]),
                                  torch.from_numpy(g[f"{tag}_row_indices"]),
                                  torch.from_numpy(g[f"{tag}_column_indices"]), O, I)
    return W, d_model, d_ff, blk, ncls


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_rmsnorm_and_mlp_outputs(case):
    g = load_golden(case)
    W, d_model, d_ff, blk, ncls = _weights(g)
    xn = orc.rmsnorm_rows(torch.from_numpy(g["x_raw"]), torch.from_numpy(g["rms_weight"]))
    np.testing.assert_allclose(xn.numpy(), g["x_normed"], rtol=2e-6, atol=1e-7)
    x = bf16_from_bits(g["x_bf16"]).float()
    y32 = orc.swiglu_mlp(x, W["gu"], W["dn"])
    np.testing.assert_allclose(y32.numpy(), g["y_fp32"], rtol=1e-5, atol=1e-7)
    yb = orc.swiglu_mlp(x, W["gu"], W["dn"], dtype=torch.bfloat16)
    np.testing.assert_array_equal(yb.view(torch.int16).numpy().astype(np.uint16), g["y_bf16"])
    gates = torch.from_numpy(g["gates_fp32"])
    yr = orc.swiglu_mlp(x, W["gu"], W["dn"], gates, ncls)
    np.testing.assert_allclose(yr.numpy(), g["y_routed_fp32"], rtol=1e-5, atol=1e-7)
    gates_ac = torch.from_numpy(g["gates_autocast"])
    yrb = orc.swiglu_mlp(x, W["gu"], W["dn"], gates_ac, ncls, dtype=torch.bfloat16)
    np.testing.assert_array_equal(yrb.view(torch.int16).numpy().astype(np.uint16),
                                  g["y_routed_bf16"])


def test_gate_formula():
    g = load_golden("mlp_tile16_d128_cs16")
    k = int(g["k"])
    gates = orc.remoe_gates(torch.from_numpy(g["router_logits"]), k)
    np.testing.assert_allclose(gates.numpy(), g["router_gates"], rtol=1e-6, atol=0)
    # the k-th largest logit maps to exactly zero: k-1 strictly active groups summing to k
    assert int((gates > 0).sum(-1).max()) == k - 1
    np.testing.assert_allclose(gates.sum(-1).numpy(), k, rtol=1e-5)


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_decode_algebra_matches_dense_path(case):
    """The decode restatement (strip layout, work-list partials, scale after the sum,
    per-stream activity flags) agrees with the reference's dense fp32 forward up to fp32
    reassociation, routed and unrouted."""
    g = load_golden(case)
    W, d_model, d_ff, blk, ncls = _weights(g)
    x = bf16_from_bits(g["x_bf16"]).float().reshape(-1, d_model)[:3]
    sp_gu = orc.pack_strips(g["gu_codes"], g["gu_column_indices"], g["gu_offsets"], g["gu_scale"])
    sp_dn = orc.pack_strips(g["dn_codes"], g["dn_column_indices"], g["dn_offsets"], g["dn_scale"])
    gates = g["gates_fp32"].reshape(-1, ncls)[:3]
    cs = d_ff // ncls
    rlo, rhi, clo, chi = orc.cluster_spans(d_ff, ncls, blk)
    ract, cact = orc.route_flags(gates, rlo, rhi, clo, chi)
    for routed in (False, True):
        kw = dict(row_act=ract, gates=gates, cluster_size=cs) if routed else {}
        h = orc.mortar_gemv(x.numpy(), sp_gu, swiglu_out=True, **kw)
        y = orc.mortar_gemv(h, sp_dn, col_act=cact if routed else None)
        # decode uses the fp32 scale, the dense path bf16(scale): compare against the
        # fp32-scale dense evaluation for tightness, and the golden output loosely.
        meta_gu = (torch.from_numpy(g["gu_row_indices"]), torch.from_numpy(g["gu_column_indices"]),
                   2 * d_ff, d_model)
        meta_dn = (torch.from_numpy(g["dn_row_indices"]), torch.from_numpy(g["dn_column_indices"]),
                   d_model, d_ff)
        yo = orc.swiglu_mlp_decode(x, torch.from_numpy(g["gu_codes"]), torch.tensor(g["gu_scale"]),
                                   meta_gu, torch.from_numpy(g["dn_codes"]),
                                   torch.tensor(g["dn_scale"]), meta_dn,
                                   torch.from_numpy(gates) if routed else None, ncls)
        scale = np.abs(yo.numpy()).max()
        assert np.abs(y - yo.numpy()).max() <= 1e-5 * scale
        ref = (g["y_routed_fp32"] if routed else g["y_fp32"]).reshape(-1, d_model)[:3]
        assert np.abs(y - ref).max() <= 2e-2 * np.abs(ref).max()


def test_router_logits_and_gates_match_reference_router():
    """The router restatement on the reference router's own parameters and input reproduces the
    logits its forward fed to topk and the gates it returned (tests/golden/make_golden.py)."""
    g = load_golden("mlp_tile16_d128_cs16")
    sd = {k[len("router_sd__"):]: v for k, v in g.items() if k.startswith("router_sd__")}
    x = bf16_from_bits(g["x_bf16"]).float().reshape(-1, 128).numpy()
    lg = orc.router_logits(x, sd["query_proj__weight"], sd["iter_embed"][0], sd["query_norm__weight"],
                           sd["query_norm__bias"], 1e-5, sd["sub_keys_a"], sd["sub_keys_b"], sd["group_bias"])
    np.testing.assert_allclose(lg, g["router_logits"], rtol=1e-5, atol=2e-6)
    k = max(1, round(0.25 * 16))
    gates = orc.remoe_gates(torch.from_numpy(g["router_logits"]), k).numpy()
    np.testing.assert_allclose(gates, g["router_gates"], rtol=1e-5, atol=1e-6)
    assert ((gates > 0).sum(axis=1) == k - 1).all()


def test_oracle_workloads_equal_the_product_generator():
    """The benchmark layers restated for the CPU baseline (which must not load the CUDA
    library) are the very matrices the product's generator makes."""
    import mortar_b200 as mb
    from oracle import workloads as wl
    for (d, f, seed) in ((768, 2048, 100), (256, 512, 7)):
        L = mb.synth.make_layer(d, f, 0.25, seed=seed)
        wg, wd, nnz = wl.dense_layer(d, f, 0.25, seed)
        assert nnz == L.gate_up.nnz + L.down.nnz
        for dense, m in ((wg, L.gate_up), (wd, L.down)):
            ref = torch.from_numpy(m.to_dense_codes()).float() * torch.tensor(m.scale)
            assert torch.equal(dense, ref)
    assert torch.equal(wl.activations(5, 64, 3), mb.synth.make_activations(5, 64, 3))


def test_decode_side_steps_against_reference_outputs():
    """hc_post and the row-scaled ternary GEMV restatements against what the reference's eager
    code produced (hc_post_reference; F.linear on the stack ternary_pack packed)."""
    from conftest import load_golden
    g = load_golden("decode_sides")
    t = lambda k: torch.from_numpy(g[k])
    out = orc.hc_post(t("hc_hres"), t("hc_hpost_row"), t("hc_h"), t("hc_y"))
    np.testing.assert_allclose(out.numpy(), g["hc_out"], rtol=1e-6, atol=1e-6)
    out = orc.hc_post(t("hc_hres"), t("hc_hpost_row"), t("hc_h"), t("hc_y"), t("hc_term"))
    np.testing.assert_allclose(out.numpy(), g["hc_out_term"], rtol=1e-6, atol=1e-6)
    y = orc.ternary_gemv_rs(g["rs_x"], g["rs_codes"], g["rs_row_scale"])
    np.testing.assert_allclose(y, g["rs_out"], rtol=2e-5, atol=1e-6)
