"""Writes the linker version script of libthnets.so from the two public headers: every function they declare, the
reference's data symbols, and nothing else (the planner, the loaders' helpers and the launch internals stay local).
Run by the Makefile whenever a header changes."""
import os
import re
import sys

here = os.path.dirname(os.path.abspath(__file__))
inc = os.path.join(here, "..", "..", "include")
names = set()
for hdr in ("thnets.h", "thb200_kernels.h"):
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(inc, hdr)).read(), flags=re.S)
    names |= set(re.findall(r"\b((?:TH|thb_|THB200_)\w+|loadtorch|freeobject|freenetwork|Module2Network|loadpytorch|"
                            r"freepynet|th_seconds)\s*\(", text))
names -= {"THB_"}
names |= {"th_debug", "th_profile", "th_minmax", "th_convtot", "th_convflops", "loadonnx"}
with open(sys.argv[1], "w") as f:
    f.write("{\n  global:\n" + "".join("    %s;\n" % n for n in sorted(names)) + "  local:\n    *;\n};\n")
