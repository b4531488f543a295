import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    return torch


@pytest.fixture(scope="session")
def moe():
    from deepstrix_b200 import moe as m
    m.lib()
    return m


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def full_mxfp4():
    """The full-size MXFP4 layer (hidden 4096, 256 + 1 experts of width 2048) resident on the GPU, built once
    per test session: generating its 3.4 GB of synthetic weights takes most of a minute.  The decode,
    prefill and mid-batch configurations share these weights, as the workload definition says."""
    import torch

    from deepstrix_b200 import moe, synth
    from deepstrix_b200.config import CONFIGS
    cfg = CONFIGS[1]
    w = synth.make_layer(cfg, 1)
    routed = moe.RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.ffn, w["gate"], w["up"], w["down"])
    shared = moe.RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.shared_ffn, w["shared_gate"], w["shared_up"], w["shared_down"])
    rw = torch.from_numpy(w["router_w"]).cuda()
    rb = torch.from_numpy(w["router_bias"]).cuda()
    yield {"cfg": cfg, "w": w, "routed": routed, "shared": shared, "rw": rw, "rb": rb}
    routed.close()
    shared.close()
