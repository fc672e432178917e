"""Host-side logic of the DDF-ResNet harness that needs no GPU: BatchNorm folding is exact.
The DDF op has no CPU path, so the oracle's unfold composite stands in for it here."""
import torch


def test_fold_batchnorm_is_exact(monkeypatch):
    import ddfnet_b200.modules as M
    from ddfnet_b200.op import spatial_filter_norm
    from ddfnet_b200.resnet import DDFResNet, fold_batchnorm
    from oracle import ddf_oracle
    monkeypatch.setattr(M, "ddf", lambda x, cf, sf, k, d, s, comb: ddf_oracle.composite_forward(
        x, cf, sf, k, d, s, comb))
    monkeypatch.setattr(M, "ddf_sfnorm", lambda x, cf, raw, k, d, s, comb, scale: ddf_oracle.composite_forward(
        x, cf, spatial_filter_norm(raw, k, scale), k, d, s, comb))
    torch.manual_seed(0)
    m = DDFResNet([1, 1, 1, 1]).double().eval()
    for mod in m.modules():
        if isinstance(mod, torch.nn.BatchNorm2d):
            mod.running_mean.normal_()
            mod.running_var.uniform_(0.5, 2)
            mod.weight.data.normal_(1, 0.2)
            mod.bias.data.normal_()
    n_bn = sum(isinstance(mod, torch.nn.BatchNorm2d) for mod in m.modules())
    x = torch.randn(2, 3, 64, 64, dtype=torch.float64)
    with torch.no_grad():
        y0 = m(x)
        fold_batchnorm(m)
        y1 = m(x)
    assert (y0 - y1).abs().max().item() <= 1e-12 * y0.abs().max().item()
    # only the BatchNorm after each DDFPack is left
    assert sum(isinstance(mod, torch.nn.BatchNorm2d) for mod in m.modules()) == 4 < n_bn
