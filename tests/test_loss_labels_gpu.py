"""Out-of-range labels on the fused loss path: skipped on the device, reported to the host, never used as an index."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_label_outside_the_class_range_is_reported_not_dereferenced():
    from scaffold_b200.ops import _lib, loss as L
    torch.manual_seed(0)
    n_classes = 5
    logits = torch.randn(1, 4, 8, 16, 8, device="cuda").to(torch.bfloat16).requires_grad_(True)
    labels = torch.randint(0, n_classes, (1, 4, 8, 16), device="cuda", dtype=torch.int16)
    cw = torch.tensor([0.5, 2.0, 2.0, 2.0, 2.0], device="cuda")
    good, _, _ = L.segmentation_loss_fused(logits, labels, n_classes, cw)
    torch.cuda.synchronize()
    _lib.check_status()
    bad = labels.clone()
    bad[0, 0, 0, 0] = 7        # a category the model does not have
    bad[0, 1, 2, 3] = -1       # an ignore value
    loss, _, _ = L.segmentation_loss_fused(logits, bad, n_classes, cw)
    loss.backward()
    torch.cuda.synchronize()
    assert torch.isfinite(loss) and torch.isfinite(logits.grad.float()).all()
    with pytest.raises(_lib.DeviceArgumentError, match="label"):
        _lib.check_status()
    # the two voxels carry no weight: the loss stays close to the clean one, and the context is usable
    assert abs(float(loss) - float(good)) < 0.05
    again, _, _ = L.segmentation_loss_fused(logits.detach(), labels, n_classes, cw)
    torch.cuda.synchronize()
    _lib.check_status()
    assert float(again) == float(good)


def test_wide_heads_take_the_framework_formula():
    from scaffold_b200.ops import loss as L
    assert L.fused_supported(32) and not L.fused_supported(33)
