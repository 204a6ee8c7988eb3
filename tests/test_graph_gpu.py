"""CUDA-graph runner with static buffers: same results as the eager public API."""
import pytest
import torch

from conftest import seeded_layer
from lowbitlinear_b200 import QuantizedLinear
from lowbitlinear_b200.graph import GraphedLinears

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [1, 4])
def test_graphed_linears_match_eager_forward(m, cuda_ops):
    shapes = [(512, 1024), (4096, 4096), (300, 768), (256, 12288), (129, 70), (1024, 256)]
    layers, inputs = [], []
    for i, (n, k) in enumerate(shapes):
        x, packed, scales, zeros = seeded_layer(m, n, k, seed=20 + i, std=0.05, device=cuda_ops)
        layers.append(QuantizedLinear(packed, scales, zeros, in_features=k))
        inputs.append(x)
    expected = [layer(x) for layer, x in zip(layers, inputs)]
    runner = GraphedLinears(layers, m=m)
    host_x = torch.zeros(runner.x_flat.numel(), dtype=torch.float16).pin_memory()
    host_y = torch.zeros(runner.y_flat.numel(), dtype=torch.float16).pin_memory()
    for offset, x in zip(runner.x_offsets, inputs):
        host_x[offset:offset + x.numel()] = x.reshape(-1).cpu()
    for _ in range(3):  # replays are repeatable
        runner.run(host_x, host_y)
        for offset, want in zip(runner.y_offsets, expected):
            got = host_y[offset:offset + want.numel()].view_as(want)
            assert torch.equal(got, want.cpu())
