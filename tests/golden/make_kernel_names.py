"""Writes kernel_names.txt: every `kernel void NAME` of the reference's Metal shaders (macro-declared
names included where the macro call spells the name), one line `file name` each.  Run where the
reference tree is present:  python tests/golden/make_kernel_names.py <reference root>."""
import os
import re
import sys


def main():
    root = sys.argv[1]
    shaders = os.path.join(root, "Resources", "Shaders")
    lines = []
    for f in sorted(os.listdir(shaders)):
        if not f.endswith(".metal"):
            continue
        text = open(os.path.join(shaders, f)).read()
        names = set(re.findall(r"^kernel void ([A-Za-z0-9_]+)", text, re.M))
        # macro instantiations: FOO(\n    name, ...) where FOO declares `kernel void NAME(`
        for macro in re.findall(r"#define ([A-Z0-9_]+)\(\s*\\?\s*NAME", text):
            names |= set(re.findall(macro + r"\(\s*([a-z][A-Za-z0-9_]+)\s*,", text))
        names.discard("NAME")
        lines += [f"{f} {n}" for n in sorted(names)]
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernel_names.txt")
    with open(out, "w") as fh:
        fh.write("\n".join(lines) + "\n")
    print(len(lines), "names ->", out)


if __name__ == "__main__":
    main()
