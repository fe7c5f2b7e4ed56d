"""The C ABI without a GPU: the library loads, exports every function include/qwenny_b200.h declares, the ctypes table
covers them all, and argument checks answer before anything touches a device."""
import os
import re

from qwenny_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    src = open(os.path.join(ROOT, "include", "qwenny_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(qb_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared()
    assert len(names) >= 40
    l = _lib.lib()
    for n in names:
        assert hasattr(l, n), f"{n} is declared but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    for n in _lib.SIGNATURES:
        assert n in names, f"{n} is bound but not declared in the header"


def test_version_and_host_only_calls():
    l = _lib.lib()
    assert b"sm_100a" in l.qb_version()
    assert l.qb_split_for(6, 5120, 16, 1024) == 40
    assert l.qb_attn_dec_splits(32005) == 36 and l.qb_attn_dec_splits(1) == 1 and l.qb_attn_dec_splits(4097) == 22
    # the same split size for every key count between two multiples of 2048 (a token's sums do not depend on the drafts
    # that follow it), never more than 37 splits (4 kv heads x 37 = one block per SM)
    for lo in range(0, 65536, 2048):
        assert all(l.qb_attn_dec_splits(k) <= 37 for k in (lo + 1, lo + 777, lo + 2048))
    # the split count follows the SM count: one block per SM over the four kv heads, 64 splits at most
    assert l.qb_attn_dec_splits_sm(32005, 148) == l.qb_attn_dec_splits(32005)
    assert l.qb_attn_dec_splits_sm(32005, 132) <= 33 and l.qb_attn_dec_splits_sm(32005, 1024) <= 64
    assert l.qb_attn_dec_splits_sm(32005, 3) >= 1


def test_argument_errors_need_no_device():
    l = _lib.lib()
    assert l.qb_row_order(17, 1, None) == 1000          # QB_ERR_ARG
    assert l.qb_marlin_gemm(None, None, None, None, None, None, 5, 256, 128, 0, 0, None, None, 0) == 1000
    assert l.qb_model_step(None, None, None, 0, None, 0) == 1000
    assert l.qb_marlin_early(None, 2) == 1000


_NULL_CALLS = """
import ctypes as C
from qwenny_b200 import _lib
l = _lib.lib()
for n in sorted(_lib.SIGNATURES):
    args = []
    for t in _lib.SIGNATURES[n]:
        if t is C.c_void_p or (isinstance(t, type) and issubclass(t, C._Pointer)):
            args.append(None)
        else:
            args.append(0.0 if t is C.c_float else 0)
    print(n, getattr(l, n)(*args), flush=True)
"""


def test_no_entry_dereferences_a_null_argument():
    """Every entry called with null pointers and zeros, in a child process (a fault there must not end the test run):
    none may crash; those that take a context, a model, a pool or a region answer QB_ERR_ARG, 0 or null."""
    import subprocess
    import sys
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-c", _NULL_CALLS], capture_output=True, text=True, timeout=300, env=env)
    seen = dict(line.split(" ", 1) for line in r.stdout.strip().splitlines())
    assert r.returncode == 0, f"crashed after {list(seen)[-1] if seen else 'nothing'}: rc {r.returncode}\n{r.stderr[-500:]}"
    assert set(seen) == set(_lib.SIGNATURES)
    free_standing = {"qb_version", "qb_static_scratch_bytes", "qb_static_device_error", "qb_step_ints"}
    for n, v in seen.items():
        if n not in free_standing:
            assert v in ("1000", "0", "None") or (n == "qb_draft_vocab_row_of" and v == "-1"), f"{n}(nulls) answered {v}"


def test_the_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: include/qwenny_b200.h compiles as C99 on its own (what a cgo / bindgen / ctypes
    binding reads), with no warnings under -Wall -Wextra -pedantic."""
    import subprocess
    src = tmp_path / "hdr.c"
    src.write_text('#include "qwenny_b200.h"\nint main(void) { return QB_OK; }\n')
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only",
                        "-I", os.path.join(ROOT, "include"), str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
