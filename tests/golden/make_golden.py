"""Regenerates the fixtures in this directory from the reference's committed outputs.

The reference runs no GEMM, so it offers no numeric golden vectors; what it pins is text:
  * tmp/log_11_18              -> bind_test_module.mlir  (stdout of test/python/bind_test.py)
  * tmp/log_12_18              -> layouts.json           (stdout of test_pass/attr_test.cpp: attribute
                                                          prints, module prints and the layout maps
                                                          GemmOp::inferLayout returned for five cases)
  * exp/layout/result/log_12_23 -> bank_stats.json       (JSON of exp/layout/gemm_layout_tool.cpp)
Run from the repository root on a machine that has the reference checked out:
    python tests/golden/make_golden.py /path/to/reference
The fixtures are data read as text; nothing of the reference is executed.
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root: str) -> None:
    with open(os.path.join(ref_root, "tmp", "log_11_18")) as f:
        module_text = f.read().rstrip("\n")
    with open(os.path.join(HERE, "bind_test_module.mlir"), "w") as f:
        f.write(module_text + "\n")

    text = open(os.path.join(ref_root, "tmp", "log_12_18")).read()
    out = {"attr_prints": re.findall(r"Constructed(?: layout)?: (\S.*?)(?: \(enum = \d+\))?$", text, re.M),
           "cases": []}
    for m in re.finditer(r"Case '(\w+)' \(target=(\w+), A=(\w+), B=(\w+)\)\n(module.*?\n\})\n(.*?)\n-{10,}|"
                         r"Case '(\w+)' \(target=(\w+), A=(\w+), B=(\w+)\)\n(module.*?\n\})\n(.*?)\n\n={10,}", text, re.S):
        g = [x for x in m.groups() if x is not None]
        name, target, a_space, b_space, module, layouts = g
        case = {"name": name, "target": target, "A": a_space, "B": b_space, "module": module, "layouts": {}}
        for lm in re.finditer(r"^(\w) layout: (\w+)\(shape=\[(\d+), (\d+)\], index=affine_map<(.*?)>"
                              r"(?:, thread=affine_map<(.*?)>, replicate=(\d+))?\)$", layouts, re.M):
            op, kind, r, c, index, thread, rep = lm.groups()
            case["layouts"][op] = {"kind": kind, "shape": [int(r), int(c)], "index": index,
                                   "thread": thread, "replicate": None if rep is None else int(rep)}
        out["cases"].append(case)
    with open(os.path.join(HERE, "layouts.json"), "w") as f:
        json.dump(out, f, indent=1)

    tool = json.load(open(os.path.join(ref_root, "exp", "layout", "result", "log_12_23")))
    stats = {"config": tool["config"],
             "layouts": [{k: l[k] for k in ("operand", "shape", "element_bits", "bank_stats",
                                            "baseline_row_major", "forward_index") if k in l}
                         for l in tool["layouts"]]}
    with open(os.path.join(HERE, "bank_stats.json"), "w") as f:
        json.dump(stats, f, indent=1)
    print(f"wrote {len(out['cases'])} layout cases, {len(stats['layouts'])} bank-stat entries")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.normpath(os.path.join(HERE, "..", "..", "..", "reference")))
