"""The C-ABI library loads and exports every symbol declared in include/clt_b200.h (no GPU needed)."""
import ctypes

from crosslayer_transcoder_b200 import _lib


def test_header_parses():
    protos = _lib.parse_header()
    assert "clt_encoder_fwd_act" in protos and "clt_adam_step" in protos
    assert len(protos) >= 18
    ret, args = protos["clt_adam_step"]
    assert ret is ctypes.c_int and len(args) == 14


def test_library_exports_every_declared_symbol():
    L = _lib.lib()                      # raises if a declared symbol is missing
    assert L.cdll.clt_version() >= 1
    for name in L.protos:
        assert hasattr(L.cdll, name)


def test_argument_errors_do_not_launch():
    L = _lib.lib()
    # bad dims are rejected before anything touches a device
    rc = L.cdll.clt_encoder_fwd_store(None, None, None, 0, 1, 1, 1, 0, None, None)
    assert rc != 0 and "bad dims" in L.last_error()


def _calls_in(path):
    """(entry point, number of arguments, line) of every ``_call("clt_...", ...)`` / ``lib().call("clt_...", ...)``
    in a Python source file, with the arguments counted at nesting depth 0."""
    import re

    text = path.read_text()
    out = []
    for m in re.finditer(r'(?:_call|\.call)\(\s*"(clt_\w+)"', text):
        i, depth, n, seen = m.end(), 0, 0, False
        while i < len(text):
            c = text[i]
            if c in "([{":
                depth += 1
            elif c in ")]}":
                if depth == 0:
                    break
                depth -= 1
            elif c == "," and depth == 0:
                n += 1
                seen = False
                i += 1
                continue
            elif c == "=" and depth == 0 and text[i + 1] != "=" and text[i - 1] not in "<>!=":
                n -= 1                      # a keyword argument of the wrapper (tag=...), not of the entry point
            if not c.isspace():
                seen = True
            i += 1
        import re as _re
        if _re.search(r",\s*\*\w", text[m.end():i]):
            continue                        # (arguments forwarded with *args cannot be counted)
        out.append((m.group(1), n if seen else n - 1, text.count("\n", 0, m.start()) + 1))
    return out


def test_host_code_calls_match_the_declared_abi():
    """Every kernel call in the host code names a declared entry point and passes as many arguments as the
    header declares (paths that only run on a GPU cannot drift from the ABI unnoticed)."""
    from pathlib import Path

    protos = _lib.parse_header()
    pkg = Path(_lib.__file__).resolve().parent
    files = [pkg / "engine.py", pkg / "data.py", pkg / "parallel.py", pkg / "model" / "clt_lightning.py"]
    n_calls = 0
    for f in files:
        for name, nargs, line in _calls_in(f):
            assert name in protos, f"{f.name}:{line}: {name} is not declared in the header"
            want = len(protos[name][1])
            assert nargs == want, f"{f.name}:{line}: {name} called with {nargs} arguments, the header declares {want}"
            n_calls += 1
    assert n_calls > 60


def test_bench_work_model_names_are_entry_points():
    """Every kernel the benchmark has a work model for is a declared entry point (a renamed or removed one would
    silently lose its roofline fraction)."""
    import importlib.util
    from pathlib import Path

    from crosslayer_transcoder_b200 import synthetic

    spec_ = importlib.util.spec_from_file_location("bench", Path(_lib.__file__).resolve().parents[1] / "bench.py")
    bench = importlib.util.module_from_spec(spec_)
    spec_.loader.exec_module(bench)
    protos = _lib.parse_header()
    for name, spec in synthetic.WORKLOADS.items():
        work = bench.algorithmic_work(bench.bench_spec(spec), 2, spec.d_features // 2, 10 ** 6, 2, nd_pad=256,
                                      fused_exchange=True)
        for k, v in work.items():
            assert k.split("[")[0] in protos, k
            assert v[0] in ("tensor", "hbm") and v[1] > 0, (name, k, v)
