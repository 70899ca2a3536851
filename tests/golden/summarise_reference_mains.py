"""Condenses the log written by tests/test_reference_mains.py (XEFUSE_REFMAINS_LOG=<file>) into the
verdict lines kept in tests/golden/reference_mains_b200.txt.

Usage: python tests/golden/summarise_reference_mains.py <log> [<out> [<environment of the test run>]]

The log holds the complete output of every reference program (tests/test_k*.cpp, the MoE examples,
the generated kernels and pipelines of IntelLabs/Xe-Fuse, built unmodified by
oracle/build_ref_mains.py) run on a B200; the summary keeps, per program, its command line, every
line that states a verdict and its exit code.
"""
import os
import re
import sys

KEEP = re.compile(r"Disposition|Passed|FAILED|Failed|PASS|FAIL|SOME_FAILED|CORRECTNESS|Correctness|"
                  r"compare: \d+ of \d+|max_rel_err")


def summarise(text):
    out = []
    for block in re.split(r"(?m)^=== (?=(?:ref_|gen_|pipe_))", text)[1:]:
        lines = block.splitlines()
        out.append("$ " + lines[0].strip())
        for ln in lines[1:]:
            if ln.startswith("rc="):
                out.append("  " + ln.strip())
            elif KEEP.search(ln) and not ln.startswith("==="):
                out.append("  " + ln.strip()[:200])
    return "\n".join(out) + "\n"


if __name__ == "__main__":
    src = sys.argv[1]
    dst = sys.argv[2] if len(sys.argv) > 2 else os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                             "reference_mains_b200.txt")
    with open(src) as f:
        body = summarise(f.read())
    env = (sys.argv[3] + " ") if len(sys.argv) > 3 else ""
    head = ("# Verdicts of the reference's own programs (IntelLabs/Xe-Fuse tests/, examples/, generated kernels and\n"
            "# pipelines; built unmodified against xe-fuse_b200/include by oracle/build_ref_mains.py) on one B200.\n"
            f"# Made by: {env}XEFUSE_REFMAINS_LOG=<log> python -m pytest tests/test_reference_mains.py -m gpu\n"
            "#          python tests/golden/summarise_reference_mains.py <log>\n")
    with open(dst, "w") as f:
        f.write(head + body)
    print(dst, body.count("$ "), "programs")
