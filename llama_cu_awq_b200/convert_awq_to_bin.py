"""Dumps every tensor of a saved AWQ state dict (torch.save'd .pt file) as raw bytes into <dir>/<key>.bin: the input
weight_packer expects (the job of the reference's convert_awq_to_bin.py).

    python -m llama_cu_awq_b200.convert_awq_to_bin <awq state dict .pt> <output dir>
"""
import os
import sys


def convert(state_path, out_dir):
    import torch
    state = torch.load(state_path, map_location="cpu")
    if not isinstance(state, dict):
        raise SystemExit(f"{state_path}: expected a dict of tensors, got {type(state).__name__}")
    os.makedirs(out_dir, exist_ok=True)
    n = 0
    for key, value in state.items():
        if not isinstance(value, torch.Tensor):
            print(key, type(value).__name__, "(skipped)")
            continue
        print(key, tuple(value.shape), value.dtype)
        with open(os.path.join(out_dir, key + ".bin"), "wb") as f:
            f.write(value.detach().cpu().contiguous().numpy().tobytes())
        n += 1
    return n


if __name__ == "__main__":
    if len(sys.argv) != 3:
        raise SystemExit(__doc__)
    convert(sys.argv[1], sys.argv[2])
