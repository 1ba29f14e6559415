"""nrl_group_advantages on the device against the oracle's restatement of the host function
(src/nn/rl.rs:436-461): bit-equal after the one rounding to f32, exact zeros for a group whose
rewards are all equal, the reference's hand values (src/nn/tests/rl.rs:550-569), and its refusals."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("groups,n", [(1, 1), (3, 2), (64, 8), (1000, 5), (7, 64)])
@pytest.mark.parametrize("norm", [dict(norm_std=False), dict(norm_std=True, eps=0.0, unbiased=True), dict(norm_std=True, eps=1e-6, unbiased=False)])
def test_bit_equal_to_the_host_function(oracle, groups, n, norm):
    from noetic_tensor_b200 import ops

    if norm.get("unbiased") and n < 2:
        pytest.skip("the sample standard deviation needs groups of at least 2")
    g = np.random.default_rng(groups * 100 + n)
    r = g.choice([0.0, 1.0], (groups, n)).astype(np.float32) if groups % 2 else g.normal(0, 3, (groups, n)).astype(np.float32)
    if groups > 2:
        r[1] = r[1, 0]  # a group with all rewards equal
    want = oracle.group_advantages(r.astype(np.float64), n, norm="std" if norm["norm_std"] else "mean", eps=norm.get("eps", 0.0), unbiased=norm.get("unbiased", True))
    got = ops.group_advantages(torch.from_numpy(r).to("cuda:0"), **norm).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.astype(np.float32).reshape(groups, n).view(np.uint32))
    if groups > 2:
        assert (got[1] == 0).all()


def test_hand_values_and_refusals():
    from noetic_tensor_b200 import capi, ops

    r = torch.tensor([[1.0, 0.0, 0.0, 1.0], [2.0, 4.0, 6.0, 8.0]], device="cuda:0")
    assert ops.group_advantages(r).cpu().tolist() == [[0.5, -0.5, -0.5, 0.5], [-3.0, -1.0, 1.0, 3.0]]
    s = ops.group_advantages(r, norm_std=True, eps=0.0, unbiased=False).cpu().numpy()
    assert np.allclose(s[0], [1, -1, -1, 1]) and np.allclose(s[1], np.array([-3, -1, 1, 3]) / np.sqrt(5.0))
    with pytest.raises(RuntimeError):
        ops.group_advantages(torch.ones(4, 1, device="cuda:0"), norm_std=True, unbiased=True)
    with pytest.raises(RuntimeError):
        ops.group_advantages(r, norm_std=True, eps=-1.0)
    assert capi.lib().nrl_group_advantages(0, 4, 0, 0.0, 0, 0, 0, None) == capi.E_BAD_ARG
