"""Install a runnable copy of the reference's Python package under baseline/_ref/ (git-ignored).

    python baseline/make_ref.py [--reference /path/to/Bi-Mamba2]

The copy is the reference's `src/ssd` tree with ONE token added: `tl.flip(..., dim=1)` in
`ssd/bi/ssd_chunk_state.py` (the installed Triton 3.x requires the argument; without it the reference's first
kernel does not compile).  Nothing under baseline/_ref is product source; it is only timed, as the Triton baseline.
"""
import argparse
import os
import shutil

HERE = os.path.dirname(os.path.abspath(__file__))


def make(reference="/root/reference"):
    src = os.path.join(reference, "src", "ssd")
    if not os.path.isdir(src):
        return None
    dst_root = os.path.join(HERE, "_ref")
    dst = os.path.join(dst_root, "ssd")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(dst_root, exist_ok=True)
    shutil.copytree(src, dst)
    path = os.path.join(dst, "bi", "ssd_chunk_state.py")
    text = open(path).read()
    needle = "tl.flip(tl.cumsum(tl.flip(dA, dim=1), axis=1))"
    if needle in text:
        text = text.replace(needle, "tl.flip(tl.cumsum(tl.flip(dA, dim=1), axis=1), dim=1)")
        open(path, "w").write(text)
    return dst


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    print(make(ap.parse_args().reference))
