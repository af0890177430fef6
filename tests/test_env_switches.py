"""Every environment switch the native sources read is documented in the C header, and every switch the
header documents is still read somewhere: a switch that nobody can find out about keeps an untested variant
alive, a documented one that is gone misleads."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "sparse_transformers_b200", "csrc")


def _read_switches():
    names = set()
    for f in os.listdir(CSRC):
        if f.endswith((".cu", ".cuh", ".cpp", ".h")):
            names |= set(re.findall(r'getenv\("(STX_[A-Z0-9_]+)"\)', open(os.path.join(CSRC, f)).read()))
    return names


def test_every_switch_is_documented_in_the_header():
    header = open(os.path.join(ROOT, "include", "stx.h")).read()
    read = _read_switches()
    assert read, "no switches found: the scan is broken"
    missing = sorted(n for n in read if n not in header)
    assert not missing, f"read by the sources but not documented in include/stx.h: {missing}"
    documented = set(re.findall(r"\b(STX_(?:STACK|PEER|ATTN)_[A-Z0-9_]+)=", header)) | set(
        re.findall(r"environment (STX_[A-Z0-9_]+)", header))
    stale = sorted(n for n in documented if n not in read)
    assert not stale, f"documented in include/stx.h but read nowhere: {stale}"
