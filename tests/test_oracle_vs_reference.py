"""The oracle against the unmodified reference modules collected under oracle/_ref, on inputs the golden files do not
hold.  Skipped where oracle/_ref has not been built (it needs the reference tree once)."""
import pytest
import torch

from oracle import build_ref
from oracle import hidream_moe_oracle as O

pytestmark = pytest.mark.skipif(not build_ref.available(), reason="oracle/_ref not built")


@pytest.mark.parametrize("n,dim,hidden_dim,e,seed", [(77, 256, 1024, 4, 11), (300, 512, 2048, 4, 12), (129, 256, 1024, 8, 13)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_matches_reference_modules(n, dim, hidden_dim, e, seed, dtype):
    from oracle import ref_runner

    layer = {k: v.to(dtype) for k, v in O.make_layer(dim, hidden_dim, e, seed=seed).items()}
    x = O.make_input(n, dim, seed=seed + 1).to(dtype)
    m = ref_runner.make_module(dim, hidden_dim, e, dtype, layer)
    with torch.no_grad():
        ref = m(x.view(1, n, dim)).view(n, dim)                       # forward as shipped: gate in x.dtype, masked branch
        idx, w, _ = m.gate(x.view(1, n, dim))
        ref_infer = m.moe_infer(x, idx.view(-1), w.view(-1, 1)) + m.shared_experts(x)
    out, oidx, ow = O.moe_layer(x, layer, gate_in_fp32=False, branch="masked")
    assert torch.equal(oidx.sort(dim=1).values, idx.sort(dim=1).values)
    out_infer, _, _ = O.moe_layer(x, layer, gate_in_fp32=False, branch="infer")
    if dtype == torch.bfloat16:
        assert torch.equal(out, ref) and torch.equal(out_infer, ref_infer)
    else:
        torch.testing.assert_close(out, ref, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(out_infer, ref_infer, rtol=1e-6, atol=1e-6)
