"""Makes tests/golden/reference_rope.safetensors: query and key vectors rotated by the
reference's OWN C++ CPU rotary kernel in its Qwen2 branch
(infMain/source/op/kernels/cpu/rope_kernel.cpp, compiled unmodified with -DQWEN2_SUPPORT
against the small stand-in header in tests/golden/cpp_shim/).

    python tests/golden/make_reference_rope_golden.py --reference /path/to/Paged-Batch-Engine

The reference's Python model (make_reference_golden.py) pairs neighbouring dimensions and
fixes theta at 1e4; its C++ engine, which is what serves Qwen2.5, pairs dimension i with
i + head_size/2 and takes theta = 1e6.  This golden pins that pairing, the direction of the
rotation and the frequency of every pair (1 / 1e6^(2i/head_size)) for the plain
implementation's ``rope_rotate_half``, at positions from 0 to a few thousand and with fewer
key heads than query heads.
"""
import argparse
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of Destination2020/Paged-Batch-Engine")
    ap.add_argument("--out", default=os.path.join(HERE, "reference_rope.safetensors"))
    args = ap.parse_args()
    cpu = os.path.join(args.reference, "infMain", "source", "op", "kernels", "cpu")
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "rope_driver")
        subprocess.run(["g++", "-O1", "-std=c++17", "-DQWEN2_SUPPORT", "-I", os.path.join(HERE, "cpp_shim"),
                        "-I", cpu, os.path.join(HERE, "rope_driver.cpp"), os.path.join(cpu, "rope_kernel.cpp"),
                        "-o", exe], check=True)
        out = {}
        for tag, (head_size, heads, kv_heads) in {"a": (16, 4, 2), "b": (48, 6, 3), "c": (128, 2, 1)}.items():
            g = torch.Generator().manual_seed(head_size)
            positions = [0, 1, 2, 7, 63, 64, 511, 2047, 4095]
            q = torch.randn(len(positions), heads * head_size, generator=g)
            k = torch.randn(len(positions), kv_heads * head_size, generator=g)
            blob = struct.pack("<4i", head_size, heads, kv_heads, len(positions))
            for i, p in enumerate(positions):
                blob += struct.pack("<i", p) + q[i].numpy().astype("<f4").tobytes() + k[i].numpy().astype("<f4").tobytes()
            res = subprocess.run([exe], input=blob, stdout=subprocess.PIPE, check=True).stdout
            per = (heads + kv_heads) * head_size
            arr = np.frombuffer(res, dtype="<f4").reshape(len(positions), per)
            out[f"{tag}.positions"] = torch.tensor(positions, dtype=torch.int32)
            out[f"{tag}.q"], out[f"{tag}.k"] = q, k
            out[f"{tag}.q_rotated"] = torch.from_numpy(arr[:, :heads * head_size].copy())
            out[f"{tag}.k_rotated"] = torch.from_numpy(arr[:, heads * head_size:].copy())
            out[f"{tag}.shape"] = torch.tensor([head_size, heads, kv_heads], dtype=torch.int32)
    from safetensors.torch import save_file
    save_file(out, args.out, metadata={"made_by": "tests/golden/make_reference_rope_golden.py",
                                       "kernel": "infMain/source/op/kernels/cpu/rope_kernel.cpp, QWEN2_SUPPORT",
                                       "theta": "1e6"})
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    sys.exit(main())
