"""Case directories for the native runner `q35run`: every tensor of one role call as raw bytes `<name>.bin` plus
`io.txt` (one line per tensor: in|out, name, dtype code, dims).  The reference keeps its kernels' test cases the same
way (a directory of `<input name>.bin` read by tools/board/axrun.cc)."""
import os

import torch

from ._lib import _DTYPE_CODE as CODE  # torch dtype -> AX dtype code


def dump_case(directory, inputs, outputs):
    """inputs / outputs: name -> tensor (any device).  Output tensors only give shapes and dtypes."""
    os.makedirs(directory, exist_ok=True)
    lines = []
    for kind, group in (("in", inputs), ("out", outputs)):
        for name, t in group.items():
            lines.append(" ".join([kind, name, str(CODE[t.dtype]), *map(str, t.shape)]))
            if kind == "in":
                t.detach().cpu().contiguous().view(torch.uint8).numpy().tofile(os.path.join(directory, name + ".bin"))
    with open(os.path.join(directory, "io.txt"), "w") as f:
        f.write("\n".join(lines) + "\n")


def read_output(directory, name, like):
    """out_<name>.bin written by q35run, as a tensor shaped and typed like `like`"""
    import numpy as np
    raw = np.fromfile(os.path.join(directory, "out_" + name + ".bin"), dtype=np.uint8)
    return torch.from_numpy(raw).view(like.dtype).reshape(like.shape)
