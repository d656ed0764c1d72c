"""Decoder-stack harness on a small configuration: the graph-replayed decode loop
must produce the same token ids as the eager loop, and a stack whose linears are
served by the W4A4 kernels must track the same stack computed with dequantised
fp16 weights and fake-quantised activations."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def small_cfg():
    from zip_kernel_b200.decoder_stack import StackConfig
    return StackConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=1000, density=0.25)


def test_graph_decode_equals_eager_decode():
    from zip_kernel_b200 import decoder_stack as ds
    dev = torch.device("cuda", 0)
    a = ds.run(small_cfg(), batch=2, prefill_len=16, decode_steps=6, device=dev, use_graph=True, seed=3)
    b = ds.run(small_cfg(), batch=2, prefill_len=16, decode_steps=6, device=dev, use_graph=False, seed=3)
    assert a["last_tokens"] == b["last_tokens"]
    assert a["value"] > 0 and a["prefill_tokens_per_s"] > 0


def test_stack_tracks_fakequant_reference(monkeypatch):
    from zip_kernel_b200 import decoder_stack as ds
    from zip_kernel_b200 import v9_linear
    dev = torch.device("cuda", 0)
    cfg = small_cfg()
    tokens = torch.randint(0, cfg.vocab, (2, 24), generator=torch.Generator().manual_seed(5)).to(dev)

    def hidden_after_prefill(forward, fused_seams=False):
        monkeypatch.setattr(ds, "v9_linear_forward", forward)
        stack = ds.DecoderStack(cfg, 2, 32, dev, seed=4, fused_seams=fused_seams)
        with torch.no_grad():
            x = stack.embed[tokens]
            for li in range(cfg.n_layers):
                x = stack._layer(li, x, 0, tokens.shape[1], None)
        return x.float()

    got = hidden_after_prefill(v9_linear.v9_linear_forward)
    ref = hidden_after_prefill(v9_linear.v9_linear_fakequant)
    rel = (got - ref).norm() / ref.norm()
    assert torch.isfinite(got).all()
    # One linear agrees with its fake-quant reference to ~4e-4 (tests of the module).  Through a
    # stack the 4-bit activation quantiser is discontinuous: a last-bit difference in a hidden state
    # flips a few codes of the next linear's input by a whole step (a step is ~15 % of the signal's
    # standard deviation), so the two stacks drift apart by a bounded fraction of that
    # quantisation noise, not by rounding error.
    assert rel.item() < 0.3, rel.item()
    # the same stack with RMSNorm and SiLU * mul fused into the quantisation launches: the fused steps round
    # exactly like their definitions, PyTorch's own RMSNorm kernel may differ from it in a last bit, and a
    # last bit can flip a 4-bit code - so the comparison is the same bounded drift, not bit equality
    fused = hidden_after_prefill(v9_linear.v9_linear_forward, fused_seams=True)
    assert torch.isfinite(fused).all()
    assert ((fused - got).norm() / got.norm()).item() < 0.3
    assert ((fused - ref).norm() / ref.norm()).item() < 0.3
