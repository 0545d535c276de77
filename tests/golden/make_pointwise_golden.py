"""Makes tests/golden/reference_pointwise.npz: RicardoMin/tiny-vLLM's own pointwise CUDA kernels.

Run by hand on a machine with a GPU, giving the folder that holds the reference's ``tinyvllm``
package (a checkout, or where it was installed):

    python tests/golden/make_pointwise_golden.py /path/to/parent/of/tinyvllm  out.npz

The reference's four pointwise operations exist as CUDA only (tinyvllm/kernels/pointwise.cu), so
the files made by make_golden.py (its model on the CPU) could not cover them.  This script
compiles the reference's three unmodified ``.cu`` files with the flags its own loader uses
(tinyvllm/kernels/_extension.py:33-42: ``-O3 -lineinfo``, not a Python module) and calls

    torch.ops.tinyvllm_cuda.rms_norm / add_rms_norm / silu_and_mul / qk_norm_rope

(tinyvllm/kernels/pointwise.py:7-55) on small random inputs in float32 and bfloat16, at a width
its kernels specialise (128, 1024) and at one they do not (48, 200).  Inputs and outputs are
saved; tests/test_plain_vs_reference.py checks that ``plain_qwen3.rms_norm``, ``add_rms_norm``,
``swiglu`` and ``qk_norm_rope`` reproduce them.

One thing is not the reference's here: its loader refuses to build unless ``nvcc --version``
names the CUDA release of the installed torch (tinyvllm/kernels/_extension.py:22-31), which no
toolkit on the machines of this project does (nvcc 12.9, torch built for 12.8); the kernels are
therefore handed to ``torch.utils.cpp_extension.load`` directly.  The kernel sources are untouched.
bfloat16 tensors are stored as float32 (exact).
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch


def build(reference_root: Path) -> None:
    from torch.utils.cpp_extension import load

    kernels = reference_root / "tinyvllm" / "kernels"
    load(name="tinyvllm_paged_decode_for_golden",
         sources=[str(kernels / name) for name in ("paged_decode.cu", "kv_store.cu", "pointwise.cu")],
         extra_cuda_cflags=["-O3", "-lineinfo"], is_python_module=False, verbose=False)


def main() -> None:
    if len(sys.argv) != 3:
        raise SystemExit("usage: make_pointwise_golden.py /path/to/parent/of/tinyvllm out.npz")
    build(Path(sys.argv[1]))
    ops = torch.ops.tinyvllm_cuda
    generator = torch.Generator().manual_seed(2024)
    saved: dict[str, np.ndarray] = {}

    def draw(*shape, spread=1.0, around=0.0):
        return around + spread * torch.randn(*shape, generator=generator)

    def keep(name: str, tensor: torch.Tensor) -> None:
        saved[name] = tensor.detach().to(torch.float32).cpu().numpy()

    for dtype, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        for width in (48, 128, 200, 1024):
            rows = 5
            x = draw(rows, width, spread=2.0).to(dtype).cuda()
            residual = draw(rows, width, spread=3.0).to(dtype).cuda()
            weight = draw(width, spread=0.1, around=1.0).to(dtype).cuda()
            for eps, eps_tag in ((1e-6, "a"), (1e-3, "b")):
                case = f"{tag}_w{width}_{eps_tag}"
                saved[f"norm_{case}_eps"] = np.asarray(eps)
                keep(f"norm_{case}_x", x), keep(f"norm_{case}_residual", residual)
                keep(f"norm_{case}_weight", weight)
                keep(f"norm_{case}_out", ops.rms_norm(x, weight, eps))
                summed_out, summed = ops.add_rms_norm(x, residual, weight, eps)
                keep(f"norm_{case}_add_out", summed_out), keep(f"norm_{case}_add_sum", summed)
        for inter in (24, 100, 3072):
            gate_up = draw(4, 2 * inter, spread=3.0).to(dtype).cuda()
            keep(f"silu_{tag}_i{inter}_x", gate_up)
            keep(f"silu_{tag}_i{inter}_out", ops.silu_and_mul(gate_up))
        for head_dim, heads, kv_heads in ((16, 4, 1), (48, 5, 5), (128, 16, 8)):
            tokens = 6
            # q and k as views into one packed projection, as the model hands them over
            # (tinyvllm/models/qwen3.py:273-293)
            packed = draw(tokens, (heads + 2 * kv_heads) * head_dim, spread=1.5).to(dtype).cuda()
            q = packed[:, :heads * head_dim].view(tokens, heads, head_dim)
            k = packed[:, heads * head_dim:(heads + kv_heads) * head_dim].view(tokens, kv_heads, head_dim)
            q_weight = draw(head_dim, spread=0.1, around=1.0).to(dtype).cuda()
            k_weight = draw(head_dim, spread=0.1, around=1.0).to(dtype).cuda()
            positions = torch.tensor([0, 1, 7, 100, 1023, 4000], dtype=torch.float32)
            inv_freq = 1.0 / (1_000_000.0 ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
            angles = torch.outer(positions, inv_freq)
            # the reference gathers float32 tables and casts them to the model dtype, [T, 1, d/2]
            # (tinyvllm/layers.py:229-245)
            cos = angles.cos().to(dtype).view(tokens, 1, head_dim // 2).cuda()
            sin = angles.sin().to(dtype).view(tokens, 1, head_dim // 2).cuda()
            eps = 1e-6
            q_out, k_out = ops.qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps, eps)
            case = f"{tag}_d{head_dim}"
            keep(f"rope_{case}_q", q), keep(f"rope_{case}_k", k)
            keep(f"rope_{case}_q_weight", q_weight), keep(f"rope_{case}_k_weight", k_weight)
            keep(f"rope_{case}_cos", angles.cos()), keep(f"rope_{case}_sin", angles.sin())
            keep(f"rope_{case}_q_out", q_out), keep(f"rope_{case}_k_out", k_out)
            saved[f"rope_{case}_eps"] = np.asarray(eps)
    torch.cuda.synchronize()
    np.savez_compressed(sys.argv[2], **saved)
    print(f"wrote {sys.argv[2]}: {len(saved)} arrays")


if __name__ == "__main__":
    main()
