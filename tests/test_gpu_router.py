"""The two-launch router (C ABI mortar_router_gates) against the router restatement and the
gates the reference router produced.  Needs a B200."""
from importlib import import_module

import numpy as np
import pytest
import torch

import mortar_b200 as mb
from conftest import bf16_from_bits, load_golden
from oracle import mortar_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
router_mod = import_module(mb.__name__ + ".router")


def _oracle_gates(x, r, it=0):
    p = {k: v.detach().cpu().numpy() for k, v in r.state_dict().items()}
    lg = orc.router_logits(x.cpu().numpy(), p["query_proj.weight"], p["iter_embed"][it], p["query_norm.weight"],
                           p["query_norm.bias"], r.query_norm.eps, p["sub_keys_a"], p["sub_keys_b"], p["group_bias"])
    return lg, orc.remoe_gates(torch.from_numpy(lg), r.activation_k).numpy()


def test_router_kernel_reproduces_reference_gates():
    g = load_golden("mlp_tile16_d128_cs16")
    r = router_mod.TileRouter(16, 128, activation_ratio=0.25)
    sd = {k[len("router_sd__"):].replace("__", "."): torch.from_numpy(v)
          for k, v in g.items() if k.startswith("router_sd__")}
    r.load_state_dict(sd)
    r = r.to(DEV).eval()
    x = bf16_from_bits(g["x_bf16"]).float().reshape(-1, 128).to(DEV)
    gates = mb.ops.router_gates(x, r)
    np.testing.assert_allclose(gates.cpu().numpy(), g["router_gates"], rtol=1e-4, atol=2e-6)
    assert np.array_equal(gates.cpu().numpy() > 0, g["router_gates"] > 0)
    # the module mirror takes the kernel path on CUDA in eval mode, leading dims preserved
    g3, aux = r(x.reshape(3, 4, 128))
    assert g3.shape == (3, 4, 16) and torch.equal(g3.reshape(-1, 16), gates)
    assert float(aux) >= 0.0


@pytest.mark.parametrize("G,nsk,ratio", [(16, 4, 0.5), (12, 4, 0.5), (40, 4, 0.25), (16, 4, 1.0), (352, 0, 0.25)])
@pytest.mark.parametrize("rows", [1, 7, 64, 300])
def test_router_kernel_all_logit_maps(G, nsk, ratio, rows):
    """1:1 product map, the G largest products (sorted), cyclic repetition, no threshold when
    k = G, and the 352-group routing of the cloud configuration (19 x 19 products)."""
    torch.manual_seed(G * 1000 + rows)
    d = 768 if G != 352 else 2048
    r = router_mod.TileRouter(G, d, activation_ratio=ratio, n_sub_keys=nsk, n_iters=3)
    with torch.no_grad():
        # without a threshold (k = G) the rule normalises relu(logits); keep its sum well away from 0
        r.group_bias.copy_(0.3 * torch.randn(G) + (3.0 if ratio >= 1.0 else 0.0))
        r.iter_embed.copy_(0.1 * torch.randn_like(r.iter_embed))
        r.query_norm.weight.copy_(1.0 + 0.1 * torch.randn(d))
        r.query_norm.bias.copy_(0.1 * torch.randn(d))
    r = r.to(DEV).eval()
    x = torch.randn(rows, d)
    gates = mb.ops.router_gates(x.to(DEV), r, iter_idx=2).cpu().numpy()
    lg, ref = _oracle_gates(x, r, it=2)
    k = r.activation_k
    np.testing.assert_allclose(gates.sum(axis=1), np.full(rows, float(k)), rtol=1e-4)
    # a logit within float noise of the threshold may flip; everything else must agree
    kth = np.sort(lg, axis=1)[:, ::-1][:, k - 1][:, None] if k < G else np.zeros((rows, 1), np.float32)
    clear = np.abs(lg - kth) > 1e-4
    assert np.array_equal((gates > 0)[clear], (ref > 0)[clear])
    np.testing.assert_allclose(gates, ref, rtol=2e-3, atol=2e-4)
    if k < G:
        assert ((gates > 0).sum(axis=1) <= k - 1 + (~clear).sum(axis=1)).all()


def test_router_kernel_rejects_bad_input():
    r = router_mod.TileRouter(16, 128).to(DEV).eval()
    with pytest.raises(ValueError):
        mb.ops.router_gates(torch.zeros(2, 64, device=DEV), r)
    with pytest.raises(NotImplementedError):
        mb.ops.router_gates(torch.zeros(2, 128), r)
    assert mb.ops.router_gates(torch.zeros(0, 128, device=DEV), r).shape == (0, 16)


def test_router_projection_paths_agree(monkeypatch):
    """Large token blocks project through a library GEMM and run only the second launch; the gates
    equal the two-launch path's up to summation order, and under autocast the projection runs in
    bf16 as the reference's nn.Linear does."""
    torch.manual_seed(5)
    r = router_mod.TileRouter(352, 2048, activation_ratio=0.25).to(DEV).eval()
    x = torch.randn(1024, 2048, device=DEV)
    n0 = mb.ops.kernel_counts().get("router", 0)
    g_gemm = mb.ops.router_gates(x, r)
    assert mb.ops.kernel_counts()["router"] - n0 == 1
    monkeypatch.setattr(mb.ops, "ROUTER_GEMM_MIN_ROWS", 1 << 30)
    g_two = mb.ops.router_gates(x, r)
    assert mb.ops.kernel_counts()["router"] - n0 == 3
    monkeypatch.undo()
    lg, _ = _oracle_gates(x.cpu(), r)
    k = r.activation_k
    kth = np.sort(lg, axis=1)[:, ::-1][:, k - 1][:, None]
    clear = torch.from_numpy(np.abs(lg - kth) > 1e-4).to(DEV)
    assert torch.equal((g_gemm > 0)[clear], (g_two > 0)[clear])
    torch.testing.assert_close(g_gemm, g_two, rtol=2e-3, atol=2e-4)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        g_ac = mb.ops.router_gates(x, r)
    q = torch.nn.functional.linear(x.bfloat16(), r.query_proj.weight.bfloat16()).float() + r.iter_embed[0]
    qn = torch.nn.functional.layer_norm(q, (2048,), r.query_norm.weight, r.query_norm.bias, r.query_norm.eps)
    sa, sb = qn[:, :1024] @ r.sub_keys_a.T, qn[:, 1024:] @ r.sub_keys_b.T
    prod = (sa.unsqueeze(2) + sb.unsqueeze(1)).reshape(1024, -1)
    lg_ac = torch.topk(prod, 352, dim=1).values + r.group_bias
    ref_ac = orc.remoe_gates(lg_ac.detach().cpu(), k).to(DEV)
    torch.testing.assert_close(g_ac, ref_ac, rtol=5e-3, atol=5e-4)
