"""GPU: the torch-extension surface (mm_amx_b200.amx_mlp), following the reference's own script
(torch-ext/test.py:14-37 check_acc shapes with integer-valued data, :122-157 Llama-7B MLP against torch)."""
import copy

import pytest
import torch

from mm_amx_b200 import amx_mlp

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(32, 32, 32), (32, 32, 4096), (512, 128, 4096)])
@pytest.mark.parametrize("device", ["cpu", "cuda"])
def test_linear_check_acc(M, N, K, device):
    torch.manual_seed(0)
    w = torch.randint(-10, 11, (N, K), dtype=torch.float32)
    x = torch.randint(-10, 11, (M, K), dtype=torch.float32)
    y0 = x @ w.T                                    # exact: small integers
    n = amx_mlp.LinearNxN()
    n.name = "fc"
    n.set_weight(w.to(torch.bfloat16).to(device))
    y1 = torch.empty((M, N), dtype=torch.float32, device=device)
    n.forward(x.to(torch.bfloat16).to(device), y1)
    assert torch.allclose(y0, y1.cpu())
    n2 = copy.deepcopy(n)
    assert n2.name == "fc"
    y2 = torch.zeros_like(y1)
    n2.forward(x.to(torch.bfloat16).to(device), y2)
    assert torch.equal(y1, y2)
    # packed weights as a tensor (torch.save-able) and back, no re-packing
    n3 = amx_mlp.LinearNxN()
    n3.load_packed_state(n.packed_state())
    y3 = torch.zeros_like(y1)
    n3.forward(x.to(torch.bfloat16).to(device), y3)
    assert torch.equal(y1, y3)


def test_linear_precondition_errors():
    n = amx_mlp.LinearNxN()
    with pytest.raises(RuntimeError):
        n.set_weight(torch.zeros(32, 32))                       # not bf16
    with pytest.raises(RuntimeError):
        n.set_weight(torch.zeros(33, 32, dtype=torch.bfloat16))  # N % 32
    n.set_weight(torch.zeros(32, 64, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        n.forward(torch.zeros(4, 32, dtype=torch.bfloat16), torch.zeros(4, 32))  # K mismatch


def test_llama_mlp_small_against_torch():
    """scaled-down version of check_acc_llama7b_MLP(M=32) (torch-ext/test.py:122-157): atol 1e-2 there."""
    torch.manual_seed(0)
    H, I, M = 512, 1408, 32
    gate, up, down = (torch.randn(I, H) * 0.05, torch.randn(I, H) * 0.05, torch.randn(H, I) * 0.05)
    x = torch.randn(M, H)
    gb, ub, db, xb = (t.to(torch.bfloat16) for t in (gate, up, down, x))
    ref = (torch.nn.functional.silu(xb.float() @ gb.float().T) * (xb.float() @ ub.float().T)).to(torch.bfloat16).float() @ db.float().T
    for device in ("cpu", "cuda"):
        mlp = amx_mlp.MLP(gb.to(device), ub.to(device), db.to(device))
        out = mlp(xb.to(device)).float().cpu()
        assert (out - ref).abs().max() <= 1e-2 * ref.abs().max()
    amx_mlp.clflush(torch.zeros(8, device="cuda"))
