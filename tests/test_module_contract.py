"""The module mirrors against the reference's module contract: constructor signatures,
``_cms`` attributes, ``state_dict`` keys in both storage flavours, and the registered
``morph_stk::dds`` operator.  Host-side only (no kernel runs here); the parts that build a
reference model run only where the reference checkout is importable."""
import inspect
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import mortar_b200 as mb
from conftest import GOLDEN_CASES, ROOT, bf16_from_bits, load_golden

# the reference checkout: MORPH_REFERENCE_ROOT, or a `reference` folder beside this repository
REF = os.environ.get("MORPH_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))
have_ref = os.path.isdir(os.path.join(REF, "morph"))


def test_constructor_signatures_match_the_reference():
    sig = inspect.signature(mb.MortarLinear.__init__)
    assert list(sig.parameters)[1:] == ["in_features", "out_features", "bias", "tile_size", "initial_density",
                                        "score_ema_alpha", "device", "dtype"]
    assert sig.parameters["bias"].default is True and sig.parameters["tile_size"].default == 16
    assert list(inspect.signature(mb.SwiGLUMortar.__init__).parameters)[1:3] == ["d_model", "d_ff"]
    lin = mb.MortarLinear(64, 128, bias=True)
    assert lin.in_features == 64 and lin.out_features == 128 and lin.tile_size == 16
    assert not lin.is_compact and lin.bias is not None and lin.bias.shape == (128,)
    lin.accumulate_scores()                                  # accepted, no-op
    with pytest.raises(RuntimeError, match="no carved weights"):
        lin.matrix
    with pytest.raises(ValueError):
        mb.MortarLinear(60, 128)
    mlp = mb.SwiGLUMortar(64, 128)
    assert mlp.gate_up.out_features == 256 and mlp.down.in_features == 128 and mlp.router is None
    assert mlp.gate_up.bias is None and mlp._last_aux_loss is None


@pytest.mark.parametrize("case", GOLDEN_CASES)
@pytest.mark.parametrize("flavour", ["packed", "unpacked"])
def test_reference_state_dict_keys_load(case, flavour):
    """The keys a carved reference model saves (block_sparse.py:783-799; packed:
    deploy_quant.py:361-365) load into a freshly constructed mirror and give the reference's
    codes and scale."""
    g = load_golden(case)
    d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])
    sd = {}
    for tag, name in (("gu", "gate_up"), ("dn", "down")):
        pre = f"{name}._cms."
        for k in ("row_indices", "column_indices", "offsets", "column_indices_t", "offsets_t", "block_offsets_t"):
            sd[pre + "mortar_" + k] = torch.from_numpy(g[f"{tag}_{k}"])
        nnz = g[f"{tag}_codes"].shape[0]
        if flavour == "packed":
            sd[pre + "mortar_packed"] = torch.from_numpy(g[f"{tag}_packed"])
            sd[pre + "mortar_scale"] = torch.tensor(float(g[f"{tag}_scale"]))
        else:
            sd[pre + "mortar_data"] = bf16_from_bits(g[f"{tag}_data_bf16"]).reshape(nnz, blk, blk)
        sd[pre + "mortar_ternary"] = torch.tensor([0.0, 0.5])
        sd[pre + "block_score_ema"] = torch.zeros(1)                    # training-side leftovers are ignored
        sd[pre + "_prune_mask"] = torch.ones(1, dtype=torch.bool)
    mlp = mb.SwiGLUMortar(d_model, d_ff)
    res = mlp.load_state_dict(sd, strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    for tag, lin, (O, I) in (("gu", mlp.gate_up, (2 * d_ff, d_model)), ("dn", mlp.down, (d_model, d_ff))):
        assert lin.is_compact and lin._cms._mortar and lin._cms._mortar_blocking == blk
        assert (lin._cms.in_features, lin._cms.out_features) == (I, O)
        direct = mb.MortarMatrix.from_reference_bcsr(g[f"{tag}_offsets"], g[f"{tag}_column_indices"],
                                                     g[f"{tag}_packed"], float(g[f"{tag}_scale"]), blk, O, I)
        np.testing.assert_array_equal(lin.matrix.codes, direct.codes)
        np.testing.assert_array_equal(lin.matrix.col_idx, direct.col_idx)
        assert np.float32(lin.matrix.scale) == np.float32(direct.scale)
        assert abs(lin.get_density() - g[f"{tag}_codes"].shape[0] / ((O // blk) * (I // blk))) < 1e-9
        with pytest.raises(AssertionError):
            lin.carve()
    # round trip through the mirror's own state_dict
    again = mb.SwiGLUMortar(d_model, d_ff)
    again.load_state_dict(mlp.state_dict())
    np.testing.assert_array_equal(again.down.matrix.codes, mlp.down.matrix.codes)
    # a dense (never carved) checkpoint is refused
    with pytest.raises(RuntimeError, match="dense"):
        mb.MortarLinear(64, 64, bias=False).load_state_dict({"_cms.weight": torch.zeros(64, 64)})


def test_state_dict_without_backward_metadata_loads():
    g = load_golden("mlp_tile16_d64")
    d_model, d_ff, blk, _ = (int(v) for v in g["meta"])
    sd = {"_cms.mortar_offsets": torch.from_numpy(g["dn_offsets"]),
          "_cms.mortar_column_indices": torch.from_numpy(g["dn_column_indices"]),
          "_cms.mortar_packed": torch.from_numpy(g["dn_packed"]),
          "_cms.mortar_scale": torch.tensor(float(g["dn_scale"]))}
    lin = mb.MortarLinear(d_ff, d_model, bias=False)
    lin.load_state_dict(sd)
    np.testing.assert_array_equal(lin._cms.mortar_row_indices.numpy(), g["dn_row_indices"])
    np.testing.assert_array_equal(lin._cms.mortar_offsets_t.numpy(), g["dn_offsets_t"])
    # the order inside a column of the transposed arrays is unspecified in the reference (argsort
    # is not declared stable): compare as sets per column
    off_t = g["dn_offsets_t"]
    for c in range(len(off_t) - 1):
        a = lin._cms.mortar_column_indices_t.numpy()[off_t[c]:off_t[c + 1]]
        assert sorted(a.tolist()) == sorted(g["dn_column_indices_t"][off_t[c]:off_t[c + 1]].tolist())


def test_morph_stk_dds_is_registered_with_the_reference_schema():
    op = torch.ops.morph_stk.dds.default
    names = [a.name for a in op._schema.arguments]
    assert names == ["lhs", "data", "offsets", "row_indices", "column_indices", "offsets_t", "column_indices_t",
                     "block_offsets_t", "shape0", "shape1", "transpose_b"]
    assert str(op._schema.returns[0].type) == "Tensor"
    # traces through fake tensors; CPU tensors are refused like the reference's CUDA-only op
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        lhs = torch.empty(256, 64, device="cuda", dtype=torch.bfloat16)
        d = torch.empty(3, 16, 16, device="cuda", dtype=torch.bfloat16)
        i16 = torch.empty(3, device="cuda", dtype=torch.int16)
        i32 = torch.empty(9, device="cuda", dtype=torch.int32)
        y = torch.ops.morph_stk.dds(lhs, d, i32, i16, i16, i32, i16, i32, 64, 128, True)
        assert y.shape == (256, 128) and y.dtype == torch.bfloat16
    with pytest.raises(NotImplementedError):
        z = torch.zeros(1, dtype=torch.int16)
        torch.ops.morph_stk.dds(torch.zeros(4, 64), torch.zeros(1, 16, 16), z.int(), z, z, z.int(), z, z.int(),
                                64, 128, True)


@pytest.mark.skipif(not have_ref, reason="reference checkout not available")
def test_reference_model_state_dict_and_op_override():
    """Build, prune, carve (and pack) a reference ``_SwiGLUMortar`` on CPU, save it, load the
    file's keys into the mirror; and with the reference imported first, its ``morph_stk::dds``
    CUDA kernel is replaced by ours."""
    code = r'''
import sys, numpy as np, torch
sys.path.insert(0, %r); sys.path.insert(0, %r)
from morph.model.transformer import _SwiGLUMortar
from morph.inference.deploy_quant import pack_mortar_ternary, _ternary_quantize
import morph.sparse.stk.backend.custom_ops          # the reference defines morph_stk::dds first
import mortar_b200 as mb
assert mb.torch_ops.install_morph_stk_dds() == "overridden"
torch.manual_seed(0)
d, f, blk = 256, 512, 128
ref = _SwiGLUMortar(d, f)
for lin in (ref.gate_up, ref.down):
    cms = lin._cms
    with torch.no_grad():
        cms.weight.copy_((torch.randn_like(cms.weight) * 0.02).to(torch.bfloat16).float())
        t = cms.tile_size
        cms.block_score_ema.copy_(cms.weight.reshape(cms.R, t, cms.C, t).pow(2).sum(dim=(1, 3)).sqrt())
    cms.prune_step_blocks(prune_rate=0.5, target_density=0.5, blocking=blk)
    cms.carve(blocking=blk)
for packed in (False, True):
    if packed:
        for lin in (ref.gate_up, ref.down):
            pack_mortar_ternary(lin._cms)
    sd = ref.state_dict()
    mir = mb.SwiGLUMortar(d, f)
    res = mir.load_state_dict(sd, strict=True)
    assert not res.missing_keys and not res.unexpected_keys, res
    for a, b in ((ref.gate_up, mir.gate_up), (ref.down, mir.down)):
        assert b.is_compact and b._cms._mortar_blocking == blk
        if packed:
            codes_ref = a._cms._mortar_effective_data().float() / a._cms.mortar_scale.to(torch.bfloat16).float()
            scale_ref = float(a._cms.mortar_scale)
        else:
            q, s = _ternary_quantize(a._cms.mortar_data.data)
            codes_ref, scale_ref = q.float(), float(s)
        m = b.matrix
        assert np.float32(m.scale) == np.float32(scale_ref)
        dense = np.zeros((a.out_features, a.in_features), dtype=np.int8)
        off = a._cms.mortar_offsets.numpy(); ci = a._cms.mortar_column_indices.numpy()
        for r in range(a.out_features // blk):
            for j in range(off[r], off[r + 1]):
                dense[r*blk:(r+1)*blk, ci[j]*blk:(ci[j]+1)*blk] = codes_ref[j].numpy().astype(np.int8)
        assert np.array_equal(m.to_dense_codes(), dense)
    # the attributes reference call sites reach through (deploy_quant.py:462-465, pruning.py:341-347)
    assert mir.gate_up._cms.in_features == d and mir.gate_up._cms.bias is None
print("OK")
''' % (REF, ROOT)
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "OK" in res.stdout, res.stdout + res.stderr
