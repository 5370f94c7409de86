"""The nn.Module layer: rank rules (CPU) and forward / backward through the fused kernels (GPU)."""
import numpy as np
import pytest
import torch

from oracle import cp_oracle as O


def test_rank_rules_follow_the_reference():
    from paralleltnnlayers_b200 import layers as L
    # generate_shape (test/layers.py:22-48)
    assert L.generate_shape(4096, base=16) == [16, 16, 16]
    assert L.generate_shape(64, base=16) == [16, 4]
    assert L.generate_shape(32, base=16) == [32]              # remainder folded into the first mode
    assert L.generate_shape(256, order=2) == [16, 16]
    assert L.generate_shape(128, order=2) == [16, 8]
    assert L.generate_shape(128, order=2, reverse=True) == [8, 16]
    with pytest.raises(ValueError):
        L.generate_shape(48, order=2)
    # generate_params_dense_cp (test/layers.py:491-507): 4096 x 4096 at rate 0.1
    p = L.params_dense_cp(4096, 4096, 0.1)
    assert p == {"input_shape": [16, 16, 16], "output_shape": [16, 16, 16], "rank": 2185}
    # generate_params_conv2d_rcp (test/layers.py:816-851): 256 -> 256, 3x3, rate 0.1
    p = L.params_conv2d_rcp(256, 256, 3, 0.1)
    assert p == {"input_shape": [16, 16], "output_shape": [16, 16], "rank": 843}
    assert L.params_conv2d_rcp(64, 64, 1, 0.5)["rank"] == int(np.ceil(0.5 * 4096 / 32))
    assert L.params_conv2d_cp4(64, 64, 3, 0.1)["rank"] == int(np.ceil(0.1 * 9 * 4096 / 134))
    assert L.params_conv2d_cp(64, 64, 3, 0.1)["rank"] == int(np.ceil(0.1 * 9 * 4096 / 137))   # test/layers.py:296-304


@pytest.mark.gpu
def test_modules_forward_backward():
    from paralleltnnlayers_b200 import layers as L
    from tests.gpu_util import check
    torch.manual_seed(0)
    # CP4
    m = L.CP4Conv2d(8, 6, 3, rank=4, bias=True).cuda()
    x = torch.randn(2, 8, 9, 10, device="cuda", requires_grad=True)
    y = m(x)
    f = [p.detach().cpu().numpy() for p in (m.FT, m.FC, m.FY, m.FX)]
    ref = O.cp4_forward(x.detach().cpu().numpy(), *f, 1) + m.bias.detach().cpu().numpy().reshape(1, -1, 1, 1)
    check(y, ref, "CP4Conv2d forward")
    dy = torch.randn_like(y)
    y.backward(dy)
    check(x.grad, O.cp4_backward_data(dy.cpu().numpy(), *f, 1), "CP4Conv2d dX")
    for p_, r in zip((m.FT, m.FC, m.FY, m.FX), O.cp4_backward_filter(x.detach().cpu().numpy(), dy.cpu().numpy(), *f, 1)):
        check(p_.grad, r, "CP4Conv2d dK", atol=1e-4)
    check(m.bias.grad, dy.sum(dim=(0, 2, 3)).cpu().numpy(), "CP4Conv2d dbias", atol=1e-4)
    # three-factor CP
    m = L.CPConv2d(8, 6, 3, rank=5).cuda()
    x = torch.randn(2, 8, 9, 10, device="cuda", requires_grad=True)
    y = m(x)
    f = [p.detach().cpu().numpy() for p in (m.KT, m.KCin, m.KC)]
    check(y, O.cp3_forward(x.detach().cpu().numpy(), *f, 1), "CPConv2d forward")
    dy = torch.randn_like(y)
    y.backward(dy)
    rX, *rK = O.cp3_backward(x.detach().cpu().numpy(), dy.cpu().numpy(), *f, 1)
    check(x.grad, rX, "CPConv2d dX")
    for p_, r in zip((m.KT, m.KCin, m.KC), rK):
        check(p_.grad, r, "CPConv2d dK", atol=1e-4)
    # rCP with the mode sizes of the rank rule
    m = L.RCPConv2d(16, 16, 3, rank=5).cuda()
    assert m.input_shape == [4, 4] and m.output_shape == [4, 4]
    x = torch.randn(2, 16, 7, 6, device="cuda", requires_grad=True)
    y = m(x)
    A = [p.detach().cpu().numpy() for p in m.factors]
    S = m.core.detach().cpu().numpy()
    check(y, O.rcp_forward(x.detach().cpu().numpy(), A, S), "RCPConv2d forward", atol=1e-4)
    dy = torch.randn_like(y)
    y.backward(dy)
    rX, rA, rS = O.rcp_backward(x.detach().cpu().numpy(), dy.cpu().numpy(), A, S)
    check(x.grad, rX, "RCPConv2d dX", atol=1e-4)
    for p_, r in zip(m.factors, rA):
        check(p_.grad, r, "RCPConv2d dA", atol=1e-4)
    check(m.core.grad, rS, "RCPConv2d dS", atol=1e-4)
    # dense
    m = L.CPDense(64, 64, rate=0.05, bias=True).cuda()
    assert m.input_shape == [16, 4] and m.output_shape == [8, 8]
    x = torch.randn(3, 5, 64, device="cuda", requires_grad=True)
    y = m(x)
    F = [p.detach().cpu().numpy() for p in m.factors]
    ref = O.dense_cp_forward(x.detach().cpu().numpy().reshape(15, 64), F).reshape(3, 5, 64) + m.bias.detach().cpu().numpy()
    check(y, ref, "CPDense forward", atol=1e-4)
    dy = torch.randn_like(y)
    y.backward(dy)
    rX, rF = O.dense_cp_backward(x.detach().cpu().numpy().reshape(15, 64), dy.cpu().numpy().reshape(15, 64), F)
    check(x.grad.reshape(15, 64), rX, "CPDense dX", atol=1e-4)
    for p_, r in zip(m.factors, rF):
        check(p_.grad, r, "CPDense dF", atol=1e-4)


def test_shape_list_reader(tmp_path):
    from paralleltnnlayers_b200.sweep import read_shapes
    f = tmp_path / "shapes.txt"
    f.write_text("# N C H W pad | T Y X\n1 256 27 27 1   384 3 3\n\n1  48 55 55 2 | 256 5 5  # comment\n1 256 27 27 1 384 3 3\n")
    assert read_shapes(str(f)) == [(1, 48, 55, 55, 2, 256, 5, 5), (1, 256, 27, 27, 1, 384, 3, 3)]


def test_shape_list_memory_table(tmp_path):
    """The KiB column of the reference's memory table: 4 * (N*T*H*W + N*C*H*W + R*(T+C+X+Y)) / 1024, floored."""
    from paralleltnnlayers_b200.sweep import main
    f = tmp_path / "shapes.txt"
    f.write_text("1 16 13 13 1 32 3 3\n")
    out = tmp_path / "m.csv"
    assert main(["--shapes", str(f), "--mem", "--ranks", "1,16", "--out", str(out)]) == 0
    kib = lambda R: 4 * (32 * 169 + 16 * 169 + R * (32 + 16 + 3 + 3)) // 1024
    assert out.read_text() == f"1 16 13 13 1 32 3 3, {kib(1)}, {kib(16)}\n"


@pytest.mark.gpu
def test_shape_list_bench_writes_the_reference_csv(tmp_path):
    import paralleltnnlayers_b200 as P
    from paralleltnnlayers_b200.sweep import bench_shapes
    f = tmp_path / "shapes.txt"
    f.write_text("1 48 27 27 2 64 5 5\n1 16 13 13 1 32 3 3\n")
    out = tmp_path / "r.csv"
    bench_shapes(P, str(f), [1, 4, 16], 3, str(out))
    rows = out.read_text().strip().split("\n")
    assert rows[0].startswith("1 16 13 13 1 32 3 3, ") and rows[1].startswith("1 48 27 27 2 64 5 5, ")
    assert all(len(r.split(", ")) == 4 and all(float(v) > 0 for v in r.split(", ")[1:]) for r in rows)


@pytest.mark.gpu
@pytest.mark.parametrize("switch", ["B200CP_STEP_NO_SHARE", "B200CP_AUTO_MMA"])
def test_layer_forward_backward_with_the_sharing_switched_off(switch):
    """The library reads its switches when it is loaded, so this runs in a fresh process: with the rank planes not
    shared (B200CP_STEP_NO_SHARE=1) or the mma path off (B200CP_AUTO_MMA=0) a CP4Conv2d layer must still run its
    forward and backward (through the plain kernels) and agree with the oracle."""
    import os
    import subprocess
    import sys
    code = r'''
import numpy as np, torch
import paralleltnnlayers_b200 as P
from oracle import cp_oracle as O
X, K0, K1, KH, KW, dU = O.make_cp4_inputs(5, 2, 8, 8, 12, 12, 3, 3, 4, factor_std=0.3)
t = [torch.from_numpy(a).cuda().requires_grad_(True) for a in (X, K0, K1, KH, KW)]
y = P.CP4Conv2dFunction.apply(*t, 1, 0)
y.backward(torch.from_numpy(dU).cuda())
ref = O.cp4_backward_filter(X, dU, K0, K1, KH, KW, 1)
assert np.allclose(y.detach().cpu().numpy(), O.cp4_forward(X, K0, K1, KH, KW, 1), rtol=1e-4, atol=1e-5)
assert np.allclose(t[0].grad.cpu().numpy(), O.cp4_backward_data(dU, K0, K1, KH, KW, 1), rtol=1e-4, atol=1e-5)
for g, r in zip(t[1:], ref):
    assert np.allclose(g.grad.cpu().numpy(), r, rtol=1e-4, atol=1e-5 * max(1.0, float(np.abs(r).max())))
print("ok")
'''
    env = dict(os.environ)
    env[switch] = "0" if switch == "B200CP_AUTO_MMA" else "1"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
