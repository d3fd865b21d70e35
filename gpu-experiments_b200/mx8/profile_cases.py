"""Small launches of the two kernels for profiler captures.

    python gpu-experiments_b200/mx8/profile_cases.py quantize [M N [launches]]
    python gpu-experiments_b200/mx8/profile_cases.py gemm [M N K [launches]]
    python gpu-experiments_b200/mx8/profile_cases.py gemm_fused [M N K [launches]]   (bf16 A quantized in the main loop)

Defaults keep the inputs larger than L2 and the device footprint well under 1 GiB so that a
multi-pass capture of one to three launches ends by itself within a minute or two.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import torch  # noqa: E402

import mx8  # noqa: E402


def main():
    what = sys.argv[1] if len(sys.argv) > 1 else "quantize"
    nums = [int(a) for a in sys.argv[2:]]
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(1)
    if what == "quantize":
        M, N = (nums + [8192, 12288])[:2] if len(nums) >= 2 else (8192, 12288)
        launches = nums[2] if len(nums) > 2 else 3
        x = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
        outs = mx8.mxfp8_quantize(x, True, True)
        for _ in range(launches - 1):
            mx8.mxfp8_quantize(x, *outs, True, True)
    else:
        M, N, K = nums[:3] if len(nums) >= 3 else (4096, 4096, 8192)
        launches = nums[3] if len(nums) > 3 else 3
        a = (torch.randn(M, K, device=dev, generator=g) * K ** -0.5).to(torch.bfloat16)
        b = (torch.randn(N, K, device=dev, generator=g) * K ** -0.5).to(torch.bfloat16)
        aq, asc, _, _ = mx8.mxfp8_quantize(a, True, False)
        bq, bsc, _, _ = mx8.mxfp8_quantize(b, True, False)
        c = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        for _ in range(launches):
            if what == "gemm_fused":
                mx8.kernel_a_bf16(a, bq, bsc, c, fused=True)
            else:
                mx8.kernel(aq, asc, bq, bsc, c)
    print("device status", mx8.device_status())


if __name__ == "__main__":
    main()
