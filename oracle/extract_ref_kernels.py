"""Writes the CUDA source the reference keeps as a Rust string constant (it compiles it at run time with NVRTC)
into oracle/_ref/, so that the Makefile can compile it for sm_100a next to the reference's .cu file.

    python oracle/extract_ref_kernels.py <reference root> <output .cu>

Only the text between  r#"  and  "#  of FUSED_OPS_KERNEL_SRC (chimere-server/src/kernels/fused_ops.rs:27-379) is
written, unchanged.  The output lives under oracle/_ref/ (git-ignored): reference sources never enter the repository."""
import os
import sys


def main():
    ref_root, out = sys.argv[1], sys.argv[2]
    src = open(os.path.join(ref_root, "chimere-server", "src", "kernels", "fused_ops.rs")).read()
    start = src.index('const FUSED_OPS_KERNEL_SRC: &str = r#"') + len('const FUSED_OPS_KERNEL_SRC: &str = r#"')
    end = src.index('"#;', start)
    os.makedirs(os.path.dirname(out), exist_ok=True)
    with open(out, "w") as f:
        f.write(src[start:end])


if __name__ == "__main__":
    main()
