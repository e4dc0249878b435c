"""``python -m dispec_b200.env_check``: prints what the engine needs to run (the role of
puneethgv/DiSpec dispec/env_check.py:15-66): torch and CUDA versions, the device, bfloat16
support, memory, the compiler, and whether the kernel libraries build and load."""
from __future__ import annotations

import shutil
import sys


def main() -> int:
    import torch

    print(f"python        {sys.version.split()[0]}")
    print(f"torch         {torch.__version__} (CUDA {torch.version.cuda})")
    ok = torch.cuda.is_available()
    print(f"cuda device   {'yes' if ok else 'NO - the engine has no CPU path'}")
    if ok:
        p = torch.cuda.get_device_properties(0)
        print(f"  name        {p.name}")
        print(f"  capability  sm_{p.major}{p.minor} ({'sm_100 family' if p.major == 10 else 'kernels are built for sm_100a only'})")
        print(f"  memory      {p.total_memory / 2**30:.1f} GiB, {p.multi_processor_count} SMs")
        print(f"  bfloat16    {torch.cuda.is_bf16_supported()}")
    print(f"nvcc          {shutil.which('nvcc') or 'not on PATH'}")
    try:
        from dispec_b200.csrc import build
        print(f"kernel lib    {build.core_library()}")
    except Exception as e:  # noqa: BLE001 - report and go on
        print(f"kernel lib    FAILED: {e}")
        return 1
    if ok:
        from dispec_b200.ops import library
        library.core()
        print("kernel lib    loaded")
    return 0


if __name__ == "__main__":
    sys.exit(main())
