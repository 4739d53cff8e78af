"""Install the UNMODIFIED reference package into baseline/_ref/ (git-ignored; it travels with a run
like the built library does) so that the benchmark can time the reference's own code paths next to
ours: its pure-PyTorch CPU path (`bench.py --impl reference`) and its Triton GPU kernels
(`secondary.reference_triton`).

    python baseline/install_ref.py /path/to/PoPE-pytorch-checkout

The reference is a pure-Python wheel (hatchling, no build step), so installing it is copying its
package directory; `pip install --no-index --target baseline/_ref` does exactly that but needs the
hatchling build backend, which is not installed here (ModuleNotFoundError: hatchling).  The one
third-party helper the reference imports and that is not installed, torch_einops_utils
(`slice_right_at_dim`, a trailing slice without arithmetic), is provided by the stand-in that also
serves the golden-vector script (tests/golden/_standin).  Nothing under baseline/_ref is committed.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def main() -> int:
    if len(sys.argv) != 2:
        print(__doc__)
        return 2
    src = os.path.join(sys.argv[1], "PoPE_pytorch")
    if not os.path.isdir(src):
        print(f"{src} not found")
        return 1
    dst_root = os.path.join(HERE, "_ref")
    os.makedirs(dst_root, exist_ok=True)
    for name, path in (("PoPE_pytorch", src),
                       ("torch_einops_utils", os.path.join(ROOT, "tests", "golden", "_standin", "torch_einops_utils"))):
        dst = os.path.join(dst_root, name)
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        shutil.copytree(path, dst, ignore=shutil.ignore_patterns("__pycache__"))
    print(f"installed PoPE_pytorch and the torch_einops_utils stand-in into {dst_root}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
