"""Layer tables of the networks the forward supports, and the tensor order of their params file.

The order mirrors the constants of nncv's tests/Nets/Res18.mlir:12-109 (what `-split-params`
walks, SplitParamsFlatArray.cpp:109-114): fc.bias, fc.weight, then the conv groups from the
last to the first of the forward pass; each group holds bn.bias, bn.weight, bn.running_var,
bn.running_mean, conv.weight.  Names are torch state-dict keys.  ResNet-50 has no fixture in
nncv; it follows torchvision's v1.5 topology with the same ordering rule.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple


@dataclass(frozen=True)
class ConvGroup:
    name: str      # state-dict prefix of the conv, e.g. "layer2.0.conv1"
    bn: str        # state-dict prefix of its batch-norm
    cin: int
    cout: int
    k: int
    stride: int
    pad: int


def conv_groups(depth: int) -> List[ConvGroup]:
    """Conv+BN groups in forward order."""
    g = [ConvGroup("conv1", "bn1", 3, 64, 7, 2, 3)]
    widths = (64, 128, 256, 512)
    if depth == 18:
        cin = 64
        for l, w in enumerate(widths):
            for b in range(2):
                stride = 2 if (b == 0 and l > 0) else 1
                p = f"layer{l + 1}.{b}"
                g.append(ConvGroup(f"{p}.conv1", f"{p}.bn1", cin, w, 3, stride, 1))
                g.append(ConvGroup(f"{p}.conv2", f"{p}.bn2", w, w, 3, 1, 1))
                if b == 0 and l > 0:
                    g.append(ConvGroup(f"{p}.downsample.0", f"{p}.downsample.1", cin, w, 1, 2, 0))
                cin = w
    elif depth == 50:
        cin = 64
        for l, (w, nb) in enumerate(zip(widths, (3, 4, 6, 3))):
            for b in range(nb):
                stride = 2 if (b == 0 and l > 0) else 1
                p = f"layer{l + 1}.{b}"
                g.append(ConvGroup(f"{p}.conv1", f"{p}.bn1", cin, w, 1, 1, 0))
                g.append(ConvGroup(f"{p}.conv2", f"{p}.bn2", w, w, 3, stride, 1))
                g.append(ConvGroup(f"{p}.conv3", f"{p}.bn3", w, 4 * w, 1, 1, 0))
                if b == 0:
                    g.append(ConvGroup(f"{p}.downsample.0", f"{p}.downsample.1", cin, 4 * w, 1, stride, 0))
                cin = 4 * w
    else:
        raise ValueError("depth must be 18 or 50")
    return g


def fc_in(depth: int) -> int:
    return 512 if depth == 18 else 2048


def tensor_order(depth: int) -> List[Tuple[str, Tuple[int, ...]]]:
    """(name, shape) of every tensor in params-file order."""
    out: List[Tuple[str, Tuple[int, ...]]] = [("fc.bias", (1000,)), ("fc.weight", (1000, fc_in(depth)))]
    for g in reversed(conv_groups(depth)):
        out += [
            (f"{g.bn}.bias", (g.cout,)),
            (f"{g.bn}.weight", (g.cout,)),
            (f"{g.bn}.running_var", (g.cout,)),
            (f"{g.bn}.running_mean", (g.cout,)),
            (f"{g.name}.weight", (g.cout, g.cin, g.k, g.k)),
        ]
    return out


def conv_macs(depth: int, h: int, w: int) -> int:
    """Direct-convolution multiply-accumulates per image (convs + FC)."""
    def out(n, g):
        return (n + 2 * g.pad - g.k) // g.stride + 1

    sizes = {}
    total = 0
    groups = conv_groups(depth)
    # spatial size entering each group: stem sees the image; blocks see the pooled map
    hh, ww = out(h, groups[0]), out(w, groups[0])
    total += hh * ww * groups[0].cout * groups[0].cin * groups[0].k ** 2
    hh, ww = (hh + 2 - 3) // 2 + 1, (ww + 2 - 3) // 2 + 1
    cur = (hh, ww)
    block_in = cur
    for g in groups[1:]:
        if g.name.endswith("conv1"):
            block_in = cur
            src = cur
        elif "downsample" in g.name:
            src = block_in
        else:
            src = cur
        oh, ow = out(src[0], g), out(src[1], g)
        total += oh * ow * g.cout * g.cin * g.k ** 2
        if "downsample" not in g.name:
            cur = (oh, ow)
        sizes[g.name] = (oh, ow)
    total += 1000 * fc_in(depth)
    return total
