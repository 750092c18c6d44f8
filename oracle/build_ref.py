"""Builds the reference's own CPU extension (its modules.cpp) into oracle/_ref
as a second checker for the oracle.  TEST INFRASTRUCTURE ONLY.

The reference sources are compiled where they lie (nothing is copied into this
repository); the one symbol its modules.cpp expects from the CUDA file that
cannot be built (cuda/dit.cu includes a header missing from the reference) is
satisfied by a stub that raises.  Output: oracle/_ref/custom_modules_ref.so.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# the reference checkout: SD3_REFERENCE_ROOT, else a directory "reference" next to this repository
REF = os.environ.get("SD3_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

STUB = r"""
#include <torch/extension.h>
#include <stdexcept>
std::vector<torch::Tensor> DiT_block_forward_cuda(
    torch::Tensor&, torch::Tensor&, torch::Tensor&,
    std::unordered_map<std::string, torch::Tensor>&,
    int, int, int, int, int, int, bool, bool, bool) {
  throw std::runtime_error("the reference's CUDA block cannot be built (missing header)");
}
"""


def build_if_possible(force=False):
    src = os.path.join(REF, "modules.cpp")
    target = os.path.join(OUT, "custom_modules_ref.so")
    if not os.path.exists(src):
        return None
    if os.path.exists(target) and not force:
        return target
    os.makedirs(OUT, exist_ok=True)
    stub = os.path.join(OUT, "cuda_stub.cpp")
    with open(stub, "w") as f:
        f.write(STUB)
    import torch
    from torch.utils import cpp_extension as ce
    inc = []
    for d in ce.include_paths():
        inc += ["-I", d]
    import sysconfig
    inc += ["-I", sysconfig.get_paths()["include"]]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w", "-DTORCH_EXTENSION_NAME=custom_modules_ref",
           "-DTORCH_API_INCLUDE_EXTENSION_H", src, stub] + inc + [
        "-L", libdir, "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-Wl,-rpath," + libdir,
        "-o", target]
    subprocess.run(cmd, check=True)
    return target


if __name__ == "__main__":
    print(build_if_possible(force="--force" in sys.argv))
