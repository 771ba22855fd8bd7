"""Host logic: canonical format, stream layout round trips, converters from the reference's
storage, metadata validation, and the C-ABI export list.  No GPU."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import mortar_b200 as mb
from conftest import GOLDEN_CASES, ROOT, bf16_from_bits, load_golden
from oracle import mortar_oracle as orc

fmt = mb.format if hasattr(mb, "format") else None
from importlib import import_module
fmt = import_module(mb.__name__ + ".format")
_lib = mb._lib


def test_abi_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "mortar_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(mortar_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.exported_symbols())


def test_status_strings_and_version():
    L = _lib.lib()
    assert b"sm_100a" in L.mortar_version()
    assert L.mortar_status_string(0) == b"ok"
    for code in range(-10, 0):
        assert L.mortar_status_string(code) != b"unknown status"


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_from_reference_storage_matches_reference_codes(case):
    g = load_golden(case)
    d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])
    for tag, (O, I) in (("gu", (2 * d_ff, d_model)), ("dn", (d_model, d_ff))):
        m = mb.MortarMatrix.from_reference_bcsr(g[f"{tag}_offsets"], g[f"{tag}_column_indices"],
                                                g[f"{tag}_packed"], float(g[f"{tag}_scale"]), blk, O, I)
        # dense code matrix rebuilt from the reference's own (unpacked) codes and indices
        ref = orc.mortar_dense(torch.from_numpy(g[f"{tag}_codes"]), torch.ones(()),
                               torch.from_numpy(g[f"{tag}_row_indices"]),
                               torch.from_numpy(g[f"{tag}_column_indices"]), O, I, False)
        np.testing.assert_array_equal(m.to_dense_codes(), ref.numpy().astype(np.int8))
        assert m.nnz == g[f"{tag}_codes"].shape[0] * (blk // 16) ** 2
        if blk == 16:   # canonical format IS the reference's flat pack at blocking 16
            np.testing.assert_array_equal(m.codes.reshape(-1), g[f"{tag}_packed"])
            np.testing.assert_array_equal(m.row_ptr, g[f"{tag}_offsets"])
            np.testing.assert_array_equal(m.col_idx, g[f"{tag}_column_indices"].astype(np.uint16))
        md = mb.MortarMatrix.from_reference_bcsr(g[f"{tag}_offsets"], g[f"{tag}_column_indices"],
                                                 g[f"{tag}_packed"], float(g[f"{tag}_scale"]), blk, O, I,
                                                 drop_zero_tiles=True)
        np.testing.assert_array_equal(md.to_dense_codes(), m.to_dense_codes())
        assert md.nnz <= m.nnz


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_from_weight_reproduces_reference_lifecycle(case):
    """topk mask + ternarise-kept-values == the reference's prune -> carve -> pack."""
    g = load_golden(case)
    d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])
    if blk != 16:
        pytest.skip("tile-granular selection only")
    from conftest import bf16_from_bits
    for tag in ("gu", "dn"):
        w = bf16_from_bits(g[f"w_{tag}_bf16"]).float()
        mask = mb.synth.topk_l2_mask(w, 0.25)
        np.testing.assert_array_equal(mask.numpy(), g[f"{tag}_prune_mask"])
        m = mb.MortarMatrix.from_weight(w, mask)
        np.testing.assert_array_equal(m.codes.reshape(-1), g[f"{tag}_packed"])
        assert np.float32(m.scale) == g[f"{tag}_scale"]


def test_stream_round_trip_ragged_and_empty_rows():
    rng = np.random.default_rng(5)
    R, C = 37, 29
    mask = rng.random((R, C)) < 0.3
    mask[3] = False            # empty row
    mask[4] = True             # full row (29 tiles: 3 full groups + 5)
    mask[5, :] = False; mask[5, 7] = True
    codes = rng.integers(-1, 2, size=(R * 16, C * 16)).astype(np.int8)
    m = mb.MortarMatrix.from_codes(codes, mask, 0.5)
    gp, gc, gcd, G = m.build_stream_host()
    assert G == sum(-(-int(n) // 8) for n in np.diff(m.row_ptr))
    assert gp[3 + 1] == gp[3]
    ci, cd = fmt.unpack_stream_host(gp, gc, gcd, m.row_ptr, m.tile_rows)
    np.testing.assert_array_equal(ci, m.col_idx)
    np.testing.assert_array_equal(cd, m.codes)
    # padding slots carry the sentinel column and all-zero codes
    cols = gc.reshape(-1, 8)
    words = gcd.view(np.uint32).reshape(-1, 32, 4)
    for r in range(R):
        n = int(m.row_ptr[r + 1] - m.row_ptr[r])
        if n % 8:
            last = gp[r + 1] - 1
            assert (cols[last, n % 8:] == 0xFFFF).all()
            for s in range(n % 8, 8):
                fields = (words[last, :, s >> 1] >> (16 * 0)) if False else words[last, :, s >> 1]
                shift = 8 * (s & 1)
                lo = (fields >> shift) & 0xFF
                hi = (fields >> (16 + shift)) & 0xFF
                assert (lo == 0x55).all() and (hi == 0x55).all()
    masked = codes.reshape(R, 16, C, 16) * mask[:, None, :, None]
    np.testing.assert_array_equal(m.to_dense_codes(), masked.reshape(R * 16, C * 16))


def test_fragment_layout_matches_mma_operand_order():
    """Lane (g,t) of a warp must find, in register i, the codes of tile elements
    (g + 8*(i&1), 2t + 8*(i>>1)) and (.., +1): the m16n8k16 A-fragment order."""
    codes = np.zeros((16, 16), dtype=np.int8)
    codes[3, 5] = 1      # g=3, t=2, low row, left half, odd column -> reg 0, high field
    codes[11, 12] = -1   # g=3, upper row, right half, t=2, even column -> reg 3, low field
    m = mb.MortarMatrix.from_codes(codes, None, 1.0)
    gp, gc, gcd, G = m.build_stream_host()
    words = gcd.view(np.uint32).reshape(G, 32, 4)
    lane = 3 * 4 + 2
    w = int(words[0, lane, 0])
    assert (w >> (2 * 0 + 16)) & 3 == 2          # stored 2 = code +1
    assert (w >> (2 * 3)) & 3 == 0               # stored 0 = code -1
    w_other = np.delete(words[0, :, 0], lane)
    assert (w_other == 0x55555555).all()


def _good():
    mask = np.array([[1, 0, 1], [0, 1, 1]], dtype=bool)
    codes = np.ones((32, 48), dtype=np.int8)
    return mb.MortarMatrix.from_codes(codes, mask, 1.0)


def test_validation_rejects_malformed_metadata():
    m = _good(); m.row_ptr = m.row_ptr.copy(); m.row_ptr[1] = 3; m.row_ptr[2] = 2
    with pytest.raises(ValueError, match="row pointer"):
        m.validate()
    m = _good(); m.row_ptr = m.row_ptr.copy(); m.row_ptr[-1] = 3
    with pytest.raises(ValueError, match="row pointer"):
        m.validate()
    m = _good(); m.col_idx = m.col_idx.copy(); m.col_idx[0] = 3
    with pytest.raises(ValueError, match="column index"):
        m.validate()
    m = _good(); m.col_idx = m.col_idx.copy(); m.col_idx[[0, 1]] = m.col_idx[[1, 0]]
    with pytest.raises(ValueError, match="column index"):
        m.validate()
    m = _good(); m.codes = m.codes.copy(); m.codes[1, 7] = 0b00001100
    with pytest.raises(ValueError, match="2-bit"):
        m.validate()
    m = _good(); m.col_idx = m.col_idx.astype(np.int32)
    with pytest.raises(ValueError, match="uint16"):
        m.validate()
    with pytest.raises(ValueError):
        mb.MortarMatrix(30, 48, np.zeros(3, np.int32), np.zeros(0, np.uint16),
                        np.zeros((0, 64), np.uint8), 1.0).validate()


def test_split_blocks_rejects_bad_input():
    g = load_golden("mlp_blk128_d256")
    off = g["gu_offsets"].copy(); off[2] = off[1] - 1
    with pytest.raises(ValueError):
        mb.MortarMatrix.from_reference_bcsr(off, g["gu_column_indices"], g["gu_packed"], 1.0, 128, 1024, 256)
    ci = g["gu_column_indices"].copy(); ci[0] = 9
    with pytest.raises(ValueError):
        mb.MortarMatrix.from_reference_bcsr(g["gu_offsets"], ci, g["gu_packed"], 1.0, 128, 1024, 256)
    with pytest.raises(ValueError):
        mb.MortarMatrix.from_reference_bcsr(g["gu_offsets"], g["gu_column_indices"], g["gu_packed"][:100],
                                            1.0, 128, 1024, 256)


def test_cpu_tensors_are_rejected_loudly():
    m = _good()
    with pytest.raises(NotImplementedError, match="CUDA-only"):
        mb.ops.act_prep(torch.zeros(2, 48))


def test_synth_generators_shapes_and_densities():
    gen = torch.Generator().manual_seed(1)
    u = mb.synth.uniform_mask(128, 352, 0.125, gen)
    assert int(u.sum()) == round(0.125 * 128 * 352)
    for rho in (0.125, 0.25, 0.5):
        z = mb.synth.zipf_row_mask(128, 352, rho, gen)
        assert abs(float(z.float().mean()) - rho) < 0.02
        # one contiguous run per row
        for r in range(0, 128, 17):
            idx = z[r].nonzero().flatten()
            if len(idx):
                assert int(idx[-1] - idx[0]) + 1 == len(idx)
    L = mb.synth.make_layer(768, 2048, 0.25, seed=100)
    assert L.gate_up.nnz == 3072 and L.down.nnz == 1536
    assert L.gate_up.algorithmic_bytes() + L.down.algorithmic_bytes() + 0 == 305360 - 0
    gates = mb.synth.make_gates(5, L, 128, 32, seed=3)
    assert int((gates > 0).sum(-1).max()) == 31
    np.testing.assert_allclose(gates.sum(-1).numpy(), 32, rtol=1e-5)
    # oracle's gate rule agrees
    lg = torch.randn(4, 16)
    np.testing.assert_array_equal(mb.synth.remoe_gates(lg, 4).numpy(), orc.remoe_gates(lg, 4).numpy())


def _unpack_row_words(words):
    """schedule row words (even columns in bits 0..15, odd columns in bits 16..31, 2 bits each)
    -> int8 codes [..., 16]"""
    w = np.asarray(words, dtype=np.uint32)
    out = np.zeros(w.shape + (16,), dtype=np.int8)
    for q in range(8):
        out[..., 2 * q] = ((w >> (2 * q)) & 3).astype(np.int8) - 1
        out[..., 2 * q + 1] = ((w >> (16 + 2 * q)) & 3).astype(np.int8) - 1
    return out


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("density", [0.35, 1.0])
def test_prefill_schedule_covers_every_tile_once(swiglu, density):
    """Replay the panel schedule on the host: summing every run's tile slots into the accumulator
    rows it names rebuilds the dense code matrix exactly -- every kept tile appears once, slots
    of rows without a kept tile hold zero codes; a panel's first run covers all 16 rows and
    overwrites, every other run accumulates; steps hold at most 48 slots and only the first
    step on a chunk fetches it."""
    rng = np.random.default_rng(3)
    R, C = (40, 23) if not swiglu else (48, 23)
    mask = rng.random((R, C)) < density
    if density < 1.0:
        mask[5] = False
        mask[6] = True
    codes = rng.integers(-1, 2, size=(R * 16, C * 16)).astype(np.int8)
    m = mb.MortarMatrix.from_codes(codes, mask, 1.0)
    h = fmt.build_sched_host(m, swiglu)
    P, CC = fmt.PANEL_ROWS, fmt.CHUNK_COLS
    units = R // 2 if swiglu else R
    per_panel = P // 2 if swiglu else P
    assert h["n_panels"] == (-(-units // per_panel) + 1) // 2 * 2     # padded to panel pairs
    assert h["n_tiles"] >= m.nnz                                      # kept tiles + zero-fill slots
    dense = np.zeros_like(codes, dtype=np.int32)
    seen = np.zeros((R, C), dtype=int)
    data = h["step_data"]
    n_slots_seen = n_live_seen = 0
    for p in range(h["n_panels"]):
        touched = 0
        started = False
        prev_chunk, prev_last = -1, True
        for st in range(h["panel_step_ptr"][p], h["panel_step_ptr"][p + 1]):
            rec = data[int(h["step_off"][st]) * 16:int(h["step_off"][st + 1]) * 16]
            hdr = rec[:16].view(np.uint32)
            n_in_step, n_runs, ck, init = (int(v) for v in hdr)
            assert ck == int(h["step_meta"][st])
            run_units = (n_runs + 7) // 8
            assert len(rec) == 16 + 16 * run_units + 64 * n_in_step
            ch, reuse, last = ck & 0x3FFF, (ck >> 30) & 1, (ck >> 31) & 1
            assert (ck >> 14) & 63 == n_in_step and (ck >> 20) & 63 == n_runs and (ck >> 29) & 1 == init
            assert reuse == (0 if prev_last else 1)
            assert ch == prev_chunk if reuse else ch > prev_chunk
            prev_chunk, prev_last = ch, bool(last)
            assert 0 <= n_in_step <= fmt.STEP_TILES == 48
            assert n_in_step > 0 or (n_runs == 0 and last and not reuse)      # mirror step of the partner
            n_slots_seen += n_in_step
            runs = rec[16:16 + 2 * n_runs].view(np.uint16).astype(int)
            tiles = _unpack_row_words(rec[16 + 16 * run_units:].view(np.uint32).reshape(n_in_step, 16))
            assert init == (1 if (n_runs and not started) else 0)
            for r in range(n_runs):
                w = int(runs[r])
                l0, first, cl, n = w & 15, (w >> 4) & 63, (w >> 10) & 3, ((w >> 12) & 15) + 1
                assert first + n <= n_in_step and l0 + n <= P
                if not started:
                    assert (l0, n) == (0, P)          # the panel's first MMA overwrites all 16 rows
                    started = True
                col = ch * CC + cl
                for k in range(n):
                    l = l0 + k
                    if swiglu:
                        half = P // 2
                        trow = p * half + l if l < half else R // 2 + p * half + (l - half)
                    else:
                        trow = p * P + l
                    t = tiles[first + k].astype(np.int32)
                    if trow >= R or not mask[trow, col]:
                        assert not t.any()           # zero-fill slot
                        continue
                    dense[trow * 16:(trow + 1) * 16, col * 16:(col + 1) * 16] += t
                    seen[trow, col] += 1
                    n_live_seen += 1
                    touched |= 1 << l
        assert prev_last
        assert touched == int(h["panel_mask"][p])
        # both panels of a pair list the same chunks
        def chunks(pp):
            return [int(h["step_meta"][st]) & 0x3FFF
                    for st in range(h["panel_step_ptr"][pp], h["panel_step_ptr"][pp + 1])
                    if not (int(h["step_meta"][st]) >> 30) & 1]
        assert chunks(p) == chunks(p ^ 1)
    assert n_slots_seen == h["n_tiles"] and n_live_seen == m.nnz
    np.testing.assert_array_equal(seen, mask.astype(int))
    np.testing.assert_array_equal(dense, m.to_dense_codes())
    if density == 1.0 and not swiglu:
        # a full panel fuses each of its columns into a single N=256 run (16 rows)
        rec0 = data[:int(h["step_off"][1]) * 16]
        assert all(((int(w) >> 12) & 15) + 1 == 16 for w in rec0[16:16 + 2 * int(rec0[4:8].view(np.uint32)[0])].view(np.uint16))


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("density", [0.35, 1.0])
def test_prefill_schedule_i8_pairs_tiles(swiglu, density):
    """The int8 schedule replayed on the host: a slot is a pair of horizontally adjacent tiles
    (16 rows x 32 columns, one nibble per code, stored value = code + 1), a chunk is four pairs;
    summing every run's slots rebuilds the dense code matrix, a missing half holds zero codes."""
    rng = np.random.default_rng(5)
    R, C = (40, 23) if not swiglu else (48, 23)          # odd column count: the last pair is half empty
    mask = rng.random((R, C)) < density
    codes = rng.integers(-1, 2, size=(R * 16, C * 16)).astype(np.int8)
    m = mb.MortarMatrix.from_codes(codes, mask, 1.0)
    h = fmt.build_sched_host(m, swiglu, arith="i8")
    P, CC = fmt.PANEL_ROWS, fmt.CHUNK_COLS
    dense = np.zeros((R * 16, (C + 1) // 2 * 32), dtype=np.int32)
    data = h["step_data"]
    for p in range(h["n_panels"]):
        started = False
        for st in range(h["panel_step_ptr"][p], h["panel_step_ptr"][p + 1]):
            rec = data[int(h["step_off"][st]) * 16:int(h["step_off"][st + 1]) * 16]
            n_in_step, n_runs, ck, init = (int(v) for v in rec[:16].view(np.uint32))
            run_units = (n_runs + 7) // 8
            assert len(rec) == 16 + 16 * run_units + 256 * n_in_step
            assert n_in_step <= 24
            ch = ck & 0x3FFF
            runs = rec[16:16 + 2 * n_runs].view(np.uint16).astype(int)
            words = rec[16 + 16 * run_units:].view(np.uint32).reshape(n_in_step, 16, 4)
            nib = np.stack([(words >> (4 * e)) & 15 for e in range(8)], axis=-1)      # [slot,row,word,8]
            assert nib.max(initial=0) <= 2
            slots = nib.reshape(n_in_step, 16, 32).astype(np.int32) - 1
            for r in range(n_runs):
                w = int(runs[r])
                l0, first, cl, n = w & 15, (w >> 4) & 63, (w >> 10) & 3, ((w >> 12) & 15) + 1
                if not started:
                    assert (l0, n) == (0, P) and init
                    started = True
                pair = ch * CC + cl
                for k in range(n):
                    l = l0 + k
                    if swiglu:
                        half = P // 2
                        trow = p * half + l if l < half else R // 2 + p * half + (l - half)
                    else:
                        trow = p * P + l
                    t = slots[first + k]
                    if trow >= R:
                        assert not t.any()
                        continue
                    dense[trow * 16:(trow + 1) * 16, pair * 32:(pair + 1) * 32] += t
    np.testing.assert_array_equal(dense[:, :C * 16], m.to_dense_codes())
    assert not dense[:, C * 16:].any()
    with pytest.raises(ValueError):
        fmt.build_sched_host(m, swiglu, arith="fp4")


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_state_dict_ingestion(case):
    """mortar_* checkpoint keys (packed and unpacked flavours) -> canonical matrix."""
    from conftest import bf16_from_bits
    g = load_golden(case)
    d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])
    for tag, (O, I) in (("gu", (2 * d_ff, d_model)), ("dn", (d_model, d_ff))):
        direct = mb.MortarMatrix.from_reference_bcsr(g[f"{tag}_offsets"], g[f"{tag}_column_indices"],
                                                     g[f"{tag}_packed"], float(g[f"{tag}_scale"]), blk, O, I)
        sd = {"mlp.x._cms.mortar_offsets": torch.from_numpy(g[f"{tag}_offsets"]),
              "mlp.x._cms.mortar_column_indices": torch.from_numpy(g[f"{tag}_column_indices"]),
              "mlp.x._cms.mortar_packed": torch.from_numpy(g[f"{tag}_packed"]),
              "mlp.x._cms.mortar_scale": torch.tensor(float(g[f"{tag}_scale"]))}
        m = mb.MortarMatrix.from_state_dict(sd, "mlp.x._cms.", O, I, blocking=blk)
        np.testing.assert_array_equal(m.codes, direct.codes)
        assert m.scale == direct.scale
        nnz = g[f"{tag}_codes"].shape[0]
        sd2 = {"p.mortar_offsets": sd["mlp.x._cms.mortar_offsets"],
               "p.mortar_column_indices": sd["mlp.x._cms.mortar_column_indices"],
               "p.mortar_data": bf16_from_bits(g[f"{tag}_data_bf16"]).reshape(nnz, blk, blk)}
        m2 = mb.MortarMatrix.from_state_dict(sd2, "p.", O, I)
        np.testing.assert_array_equal(m2.codes, direct.codes)
        assert np.float32(m2.scale) == np.float32(direct.scale)
    with pytest.raises(KeyError):
        mb.MortarMatrix.from_state_dict({}, "p.", 64, 64)


def test_router_mirror_matches_reference_gates():
    """The TileRouter mirror takes the reference router's own ``state_dict`` (same names and
    shapes); on those parameters the router restatement reproduces the reference's logits and
    gates, and the mirror itself has no CPU evaluation."""
    from importlib import import_module
    from conftest import bf16_from_bits
    router = import_module(mb.__name__ + ".router")
    g = load_golden("mlp_tile16_d128_cs16")
    r = router.TileRouter(16, 128, activation_ratio=0.25)
    assert r.activation_k == int(g["k"]) and r.n_sub_keys == 4
    sd = {k[len("router_sd__"):].replace("__", "."): torch.from_numpy(v)
          for k, v in g.items() if k.startswith("router_sd__")}
    assert set(sd) == set(r.state_dict())
    r.load_state_dict(sd)
    r.eval()
    x = bf16_from_bits(g["x_bf16"]).float().reshape(-1, 128)
    p = {k: v.numpy() for k, v in sd.items()}
    logits = orc.router_logits(x.numpy(), p["query_proj.weight"], p["iter_embed"][0], p["query_norm.weight"],
                               p["query_norm.bias"], r.query_norm.eps, p["sub_keys_a"], p["sub_keys_b"],
                               p["group_bias"])
    gates = orc.remoe_gates(torch.from_numpy(logits), r.activation_k)
    np.testing.assert_allclose(logits, g["router_logits"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(gates.numpy(), g["router_gates"], rtol=1e-4, atol=1e-6)
    with pytest.raises(NotImplementedError):
        r(x)


def test_custom_ops_have_fake_kernels_and_no_cpu_path():
    """The registered ops trace through fake tensors (shapes and dtypes only) and refuse CPU
    tensors the way the reference's CUDA-only operator does."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(3, 5, 64, device="cuda", dtype=torch.bfloat16)
        gp = torch.empty(9, device="cuda", dtype=torch.int32)
        gc = torch.empty(10, 8, device="cuda", dtype=torch.int16)
        gk = torch.empty(10, 512, device="cuda", dtype=torch.uint8)
        y = torch.ops.mortar_b200.linear(x, gp, gc, gk, 0.5, 128, 64, 10)
        assert y.shape == (3, 5, 128) and y.dtype == torch.bfloat16 and y.device.type == "cuda"
        y = torch.ops.mortar_b200.mlp_prefill(x, gp, gc, gk, 0.5, 256, 64, 10, gp, gc, gk, 0.5, 64, 128, 10, None, 0)
        assert y.shape == (3, 5, 64) and y.dtype == torch.bfloat16
        xf = torch.empty(7, 64, device="cuda", dtype=torch.float32)
        y = torch.ops.mortar_b200.mlp_decode(xf, None, 1e-6, gp, gc, gk, 0.5, 256, 64, 10, gp, gc, gk, 0.5, 64, 128,
                                             10, None, 0)
        assert y.shape == (7, 64) and y.dtype == torch.float32
    with pytest.raises(NotImplementedError):
        torch.ops.mortar_b200.linear(torch.zeros(2, 64), torch.zeros(9, dtype=torch.int32),
                                     torch.zeros(1, 8, dtype=torch.int16), torch.zeros(1, 512, dtype=torch.uint8),
                                     0.5, 128, 64, 1)
    with pytest.raises(NotImplementedError):
        z = torch.zeros(1)
        mb.torch_ops.stk_dds(torch.zeros(2, 64), z, z, z, z, z, z, z, 64, 128, True)


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_dds_shim_conversion_of_effective_weights(case):
    """[nnz, blk, blk] effective weights (code * bf16 scale, what a ternarised layer feeds the
    reference operator) + the reference's row pointers / column ids -> the same tiles as the
    packed-storage converter; anything that is not ternary is refused."""
    g = load_golden(case)
    d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])
    for tag, (O, I) in (("gu", (2 * d_ff, d_model)), ("dn", (d_model, d_ff))):
        sc = torch.tensor(float(g[f"{tag}_scale"])).to(torch.bfloat16)
        data = (torch.from_numpy(g[f"{tag}_codes"]).float() * sc.float()).to(torch.bfloat16)
        m = mb.torch_ops._ternary_matrix_from_data(data, torch.from_numpy(g[f"{tag}_offsets"]),
                                                   torch.from_numpy(g[f"{tag}_column_indices"]), O, I)
        ref = mb.MortarMatrix.from_reference_bcsr(g[f"{tag}_offsets"], g[f"{tag}_column_indices"],
                                                  g[f"{tag}_packed"], float(g[f"{tag}_scale"]), blk, O, I)
        np.testing.assert_array_equal(m.to_dense_codes(), ref.to_dense_codes())
        assert m.scale == float(sc)
        raw = bf16_from_bits(g[f"{tag}_data_bf16"])          # the un-ternarised carved weights
        with pytest.raises(ValueError):
            mb.torch_ops._ternary_matrix_from_data(raw, torch.from_numpy(g[f"{tag}_offsets"]),
                                                   torch.from_numpy(g[f"{tag}_column_indices"]), O, I)
