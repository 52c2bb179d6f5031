"""B200-native adder convolution (AdderNet) behind the API of LingYeAI/AdderNetCUDA.

    import addernetcuda_b200 as ab
    ab.install_dropin()          # makes `import adder` / `import adder_cuda` resolve to this package
    import resnet20              # the reference's model file, unchanged

Sub-modules: `adder` (adder2d, adder2d_function, adder), `adder_cuda` (the extension's entry
points plus the fused forward/backward), `resnet` (ResNet-20/50 builders), `ddp` (bucketed
gradient all-reduce for batch-sharded training), `build` (nvcc build of the C-ABI library).
"""
import sys as _sys

__version__ = "0.1.0"


def install_dropin() -> None:
    """Register this package's `adder` and `adder_cuda` under the reference's top-level names."""
    from . import adder as _adder, adder_cuda as _adder_cuda
    _sys.modules["adder"] = _adder
    _sys.modules["adder_cuda"] = _adder_cuda


def strict_fp32() -> None:
    """Make the multiply-based layers around the adder layers (stem convolution, 1x1 `fc`) compute in
    true fp32: PyTorch lets cuDNN use TF32 for convolutions by default, which alone moves ResNet-20
    logits by ~5e-3 relative to the fp32 reference.  The adder kernels themselves are always fp32."""
    import torch
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
