"""Parameter shapes of ResNet-50 (25.6 M parameters in conv / batch-norm / fc
layers), built from the architecture's definition: the gradient-bucket workload
allreduces one gradient tensor per parameter.  No weights are needed."""
from __future__ import annotations

import torch


def resnet50_param_shapes() -> list[tuple[str, tuple[int, ...]]]:
    """``[(name, shape), ...]`` in the order ``torchvision.models.resnet50().named_parameters()`` yields them."""
    shapes: list[tuple[str, tuple[int, ...]]] = []

    def conv(name, cout, cin, k):
        shapes.append((f"{name}.weight", (cout, cin, k, k)))

    def bn(name, c):
        shapes.append((f"{name}.weight", (c,)))
        shapes.append((f"{name}.bias", (c,)))

    conv("conv1", 64, 3, 7)
    bn("bn1", 64)
    inplanes = 64
    for li, (planes, blocks) in enumerate(((64, 3), (128, 4), (256, 6), (512, 3)), start=1):
        for b in range(blocks):
            p = f"layer{li}.{b}"
            conv(f"{p}.conv1", planes, inplanes, 1)
            bn(f"{p}.bn1", planes)
            conv(f"{p}.conv2", planes, planes, 3)
            bn(f"{p}.bn2", planes)
            conv(f"{p}.conv3", planes * 4, planes, 1)
            bn(f"{p}.bn3", planes * 4)
            if b == 0:
                conv(f"{p}.downsample.0", planes * 4, inplanes, 1)
                bn(f"{p}.downsample.1", planes * 4)
            inplanes = planes * 4
    shapes.append(("fc.weight", (1000, 2048)))
    shapes.append(("fc.bias", (1000,)))
    return shapes


def resnet50_num_params() -> int:
    n = 0
    for _, s in resnet50_param_shapes():
        k = 1
        for d in s:
            k *= d
        n += k
    return n


def synthetic_grads(device, dtype=torch.float32, seed: int = 0, std: float = 1e-3) -> list[torch.Tensor]:
    """Random-init gradients ~ N(0, std^2) in ResNet-50's parameter shapes."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return [torch.randn(s, device=device, dtype=torch.float32, generator=g).mul_(std).to(dtype) for _, s in resnet50_param_shapes()]
