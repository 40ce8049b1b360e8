"""The Python side declares each kernel entry point's argument types by hand; a count that differs from
the C prototype would shift the stream pointer.  This compares the two without a GPU."""
import re
from pathlib import Path

from gpullama3.java_b200.kernels import ops

CSRC = Path(ops.__file__).resolve().parent.parent / "csrc"


def c_parameters(source: str, name: str) -> list[str]:
    m = re.search(r'extern\s+"C"\s+int\s+' + re.escape(name) + r"\s*\(", source)
    assert m, f"{name} has no extern \"C\" definition"
    depth, i = 1, m.end()
    while depth:
        depth += {"(": 1, ")": -1}.get(source[i], 0)
        i += 1
    return [p.strip() for p in source[m.end():i - 1].split(",")]


def test_declared_argument_counts_match_the_c_prototypes():
    for name, (lib, argtypes) in ops._SIGNATURES.items():
        params = c_parameters((CSRC / f"{lib}.cu").read_text(), name)
        assert params[-1].startswith("cudaStream_t"), (name, params[-1])
        assert len(params) == len(argtypes) + 1, f"{name}: C takes {len(params)}, Python declares {len(argtypes) + 1}"
        for p, t in zip(params, argtypes):  # pointers are declared as pointers, scalars as scalars
            assert ("*" in p) == (t is ops.c_void_p), (name, p, t)
