"""Operator front ends on the PyTorch path (CPU): options that the GPU tests check against the kernels."""


def test_linear_cross_entropy_label_smoothing_and_softcap_reference():
    import torch
    from pmetal_b200.ops import functional as F
    torch.manual_seed(0)
    h, w = torch.randn(37, 16), torch.randn(50, 16)
    lab = torch.randint(0, 50, (37,))
    lab[::4] = -100
    s, n = F.linear_cross_entropy(h, w, lab, softcap=5.0, label_smoothing=0.2, chunk=16)
    lg = 5.0 * torch.tanh((h @ w.t()) / 5.0)
    want = torch.nn.functional.cross_entropy(lg, lab, ignore_index=-100, reduction="sum", label_smoothing=0.2)
    assert abs(float(s) - float(want)) < 1e-3 and int(n) == int((lab != -100).sum())
