"""Second, independent CPU check of the oracle: the same networks written with PyTorch's CPU
operators (fp32).  Used only to validate oracle/nncv_oracle.cpp."""
import torch
import torch.nn.functional as F

from nncv_b200.netspec import conv_groups


def resnet_forward(depth, x, sd, dtype=torch.float32):
    t = {k: torch.from_numpy(v).to(dtype) for k, v in sd.items()}
    x = torch.from_numpy(x).to(dtype)

    def cbr(x, g, relu):
        y = F.conv2d(x, t[f"{g.name}.weight"], stride=g.stride, padding=g.pad)
        y = F.batch_norm(y, t[f"{g.bn}.running_mean"], t[f"{g.bn}.running_var"], t[f"{g.bn}.weight"],
                         t[f"{g.bn}.bias"], training=False, eps=1e-5)
        return F.relu(y) if relu else y

    groups = {g.name: g for g in conv_groups(depth)}
    x = cbr(x, groups["conv1"], True)
    x = F.max_pool2d(x, 3, 2, 1)
    nblocks = (2, 2, 2, 2) if depth == 18 else (3, 4, 6, 3)
    for l in range(4):
        for b in range(nblocks[l]):
            p = f"layer{l + 1}.{b}"
            y = cbr(x, groups[f"{p}.conv1"], True)
            if depth == 18:
                y = cbr(y, groups[f"{p}.conv2"], False)
            else:
                y = cbr(y, groups[f"{p}.conv2"], True)
                y = cbr(y, groups[f"{p}.conv3"], False)
            idn = cbr(x, groups[f"{p}.downsample.0"], False) if f"{p}.downsample.0" in groups else x
            x = F.relu(y + idn)
    x = x.mean(dim=(2, 3))
    return (x @ t["fc.weight"].T + t["fc.bias"]).numpy()
