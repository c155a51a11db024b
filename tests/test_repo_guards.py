"""Repository guards (the reference keeps the same kind under scripts/: dependency direction, no baked paths;
website/docs/develop/test.md:78-89): layering of the package, nothing in the product depends on scratch folders or
on the test-only kernel emulation, sources carry no machine paths, every registered kernel signature is exported by
a CUDA source, and every closed-call name stays out of the tree."""
import ast
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "poot_b200")

# a package may import the packages listed for it (and itself); lower layers never reach up
LAYERS = {
    "tensor": set(), "target": {"tensor"}, "quant": {"tensor", "ops"}, "weights": {"tensor", "quant"},
    "load": {"tensor", "quant", "weights", "models"}, "ir": {"tensor", "quant"}, "oracle": {"tensor", "quant", "ir", "models", "runtime", "ops"},
    "models": {"tensor", "ir", "load", "quant"}, "plan": {"tensor", "ir", "quant", "target", "models", "oracle"},
    "ops": set(), "profile": {"target", "ops"}, "text": {"ops"},
    "runtime": {"models", "ops", "quant", "parallel", "tensor", "plan"}, "parallel": {"ops", "runtime"},
    "utils": {"ops", "oracle", "runtime", "models", "tensor", "plan", "quant"},
    "driver": {"models", "runtime", "ops", "load", "quant", "ir", "oracle", "text", "tensor", "profile", "parallel", "plan"},
    "serve": {"driver", "text", "profile", "models", "parallel", "runtime", "ops", "load", "plan"}, "cli": {"driver", "text", "models", "plan", "load"},
}
TOP = {"llm": None, "embed": None, "vlm": None, "build": None, "__init__": None}     # facades at the package root may import anything


def _py_files(base):
    for d, dirs, files in os.walk(base):
        dirs[:] = [x for x in dirs if x not in ("__pycache__", "lib")]
        for f in files:
            if f.endswith(".py"):
                yield os.path.join(d, f)


def _imports(path):
    tree = ast.parse(open(path).read(), path)
    rel = os.path.relpath(path, PKG).split(os.sep)
    for node in ast.walk(tree):
        if isinstance(node, ast.ImportFrom):
            if node.level:           # relative: resolve against the file's package
                base = rel[:-1]
                up = node.level - 1
                base = base[:len(base) - up] if up else base
                mod = base + (node.module.split(".") if node.module else [])
                yield ".".join(["poot_b200"] + mod)
            elif node.module:
                yield node.module
        elif isinstance(node, ast.Import):
            for a in node.names:
                yield a.name


def test_package_layering():
    bad = []
    for path in _py_files(PKG):
        rel = os.path.relpath(path, PKG).split(os.sep)
        me = rel[0] if len(rel) > 1 else rel[0][:-3]
        if me in TOP:
            continue
        assert me in LAYERS, f"package {me!r} is not in the layer table"
        for mod in _imports(path):
            parts = mod.split(".")
            if parts[0] != "poot_b200" or len(parts) < 2:
                continue
            dep = parts[1]
            if dep == me or dep in TOP and dep != "__init__":
                if dep in ("llm", "embed", "vlm") and me != "cli" and me != "serve":
                    bad.append((os.path.relpath(path, ROOT), mod))
                continue
            if dep not in LAYERS[me]:
                bad.append((os.path.relpath(path, ROOT), mod))
    assert not bad, bad


def test_product_does_not_depend_on_scratch_or_on_the_kernel_emulation():
    for path in list(_py_files(PKG)) + [os.path.join(ROOT, "bench.py"), os.path.join(ROOT, "__graft_entry__.py")]:
        src = open(path).read()
        assert not re.search(r"(^|[^a-z])_work([^a-z]|$)", src), path
        if not path.endswith((os.path.join("utils", "kernel_emulation.py"), os.path.join("utils", "tp_emulation.py"))):
            assert "kernel_emulation" not in src and "tp_emulation" not in src, f"{path}: the host emulation is a test harness, nothing in the product selects it"


def test_sources_carry_no_machine_paths_or_closed_calls():
    # the patterns are assembled from pieces so that this file does not itself contain what it looks for
    batch = "Batch" + "Async"
    pat = re.compile("/ro" + "ot/|/ho" + "me/[a-z]|cudaMemcpy(3D)?" + batch + "|cuMemcpy(3D)?" + batch + "|multi" + "cast::clu" + "ster")
    hits = []
    for base, exts in ((PKG, (".py",)), (os.path.join(ROOT, "csrc"), (".cu", ".cuh", ".cpp", ".h")),
                       (os.path.join(ROOT, "benchmarks"), (".py",)), (os.path.join(ROOT, "tests"), (".py",))):
        for d, dirs, files in os.walk(base):
            dirs[:] = [x for x in dirs if x != "__pycache__"]
            for f in files:
                if f.endswith(exts) and f != "test_repo_guards.py":
                    for i, line in enumerate(open(os.path.join(d, f), errors="replace"), 1):
                        if pat.search(line):
                            hits.append((os.path.relpath(os.path.join(d, f), ROOT), i, line.strip()[:80]))
    assert not hits, hits


def test_every_registered_kernel_entry_is_exported_by_a_source():
    from poot_b200.ops import cuda_ops, moe_ops, suffix_ops  # noqa: F401  (registration happens at import)
    names = set(cuda_ops._SIGS) if hasattr(cuda_ops, "_SIGS") else set()
    exported = set()
    for d, _, files in os.walk(os.path.join(ROOT, "csrc")):
        for f in files:
            if f.endswith((".cu", ".cpp")):
                exported |= set(re.findall(r"POOT_API\s+[\w\s\*]+?\b(poot_\w+)\s*\(", open(os.path.join(d, f)).read()))
    assert names, "the signature table was not found"
    missing = sorted(n for n in names if n not in exported)
    assert not missing, missing


def test_ctypes_signatures_match_the_c_declarations():
    """Every registered ctypes signature has the parameter kinds, in order, of the exported C function: a pointer (or
    stream) for a pointer, ``int`` / ``long long`` / ``float`` for themselves.  A kernel entry whose argument list
    changed without its binding (or the other way round) fails here, not on a device."""
    import ctypes
    from poot_b200.ops import cuda_ops, moe_ops, suffix_ops  # noqa: F401
    from poot_b200.parallel import tp  # noqa: F401  (registers the comm launchers)
    decl = {}
    for d, _, files in os.walk(os.path.join(ROOT, "csrc", "kernels")):
        for f in files:
            if f.endswith(".cu"):
                src = open(os.path.join(d, f)).read()
                for m in re.finditer(r"POOT_API\s+int\s+(poot_\w+)\s*\(([^)]*)\)", src):
                    decl[m.group(1)] = m.group(2)

    def kind(param: str):
        p = param.strip()
        if "*" in p or p.startswith("cudaStream_t"):
            return ctypes.c_void_p
        base = re.sub(r"\b(const|unsigned)\b", "", p).split()
        ty = " ".join(base[:-1]) if len(base) > 1 else base[0]
        return {"int": ctypes.c_int, "long long": ctypes.c_longlong, "float": ctypes.c_float, "size_t": ctypes.c_size_t,
                "uint32_t": ctypes.c_uint32}.get(ty, ty)

    bad = []
    for name, sig in cuda_ops._SIGS.items():
        if name not in decl:
            continue                       # exported-by-a-source is checked above
        want = [kind(p) for p in decl[name].split(",") if p.strip()]
        if list(sig) != want:
            bad.append((name, [getattr(t, "__name__", t) for t in sig], [getattr(t, "__name__", t) for t in want]))
    assert not bad, bad


def test_every_typed_error_is_named_by_a_test():
    """Variant coverage: an exception class the package defines must appear by name in some test, so a refusal or
    failure path nobody exercises cannot be added silently (the reference's ``scripts/check-variant-coverage.py``)."""
    import re
    pat = re.compile(r"(Error|Exception|Refus\w*|Unavailable|Incompatible|Fault|Timeout|Lost|Failed|Missing|Overrun|"
                     r"NeedsReset|Poisoned|Validation|OutOfRange|TooSmall|Exceeded|Layout)$")
    classes = {}
    for path in _py_files(PKG):
        for node in ast.walk(ast.parse(open(path).read(), path)):
            if isinstance(node, ast.ClassDef) and pat.search(node.name) and node.bases:
                classes[node.name] = os.path.relpath(path, ROOT)
    here = os.path.dirname(__file__)
    tests = "".join(open(os.path.join(here, f)).read() for f in os.listdir(here) if f.endswith(".py"))
    missing = sorted((c, p) for c, p in classes.items() if not re.search(r"\b" + c + r"\b", tests))
    assert len(classes) > 30 and not missing, missing
