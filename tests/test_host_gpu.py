"""The host-buffer front end gives the same bits as the device-pointer operators."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_host_linear_equals_device_path():
    from inference_b200 import ops, synth
    from inference_b200.host import HostLinearFP8
    m, n, k = 1000, 640, 1024   # several panels, the last one ragged
    x = synth.activations(m, k, seed=4)
    bq, bs = synth.quantised_weights(n, k, seed=4)
    aq, a_s = ops.quant_fp8_per_token_group(x)
    want = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.bfloat16).cpu()
    lin = HostLinearFP8(bq, bs, max_rows=m, panel_rows=256)
    x_host = x.cpu().pin_memory()
    out = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
    for _ in range(2):   # buffers are reused across calls
        out.fill_(0)
        lin(x_host, out)
        assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    assert ops.device_status()[0] == 0
