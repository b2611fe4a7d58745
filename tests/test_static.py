"""Static checks over the whole source tree (no GPU, nothing imported): every global name a function loads is
defined in its module or is a builtin, and every kernel operator the Python side calls has a schema in the
bindings. They cover the branches that only run on GPUs, which the CPU suite never executes."""
import ast
import builtins
import dis
import os
import re
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TREES = ["oslo_b200", "examples", "tests", "baseline/reference_runner.py", "bench.py", "__graft_entry__.py", "setup.py"]


def _files():
    for t in TREES:
        p = os.path.join(ROOT, t)
        if p.endswith(".py"):
            yield p
            continue
        for d, _, fs in os.walk(p):
            if "__pycache__" in d:
                continue
            for f in fs:
                if f.endswith(".py"):
                    yield os.path.join(d, f)


def _module_names(tree):
    names = set()
    for node in ast.walk(tree):
        if isinstance(node, (ast.Import, ast.ImportFrom)):
            names.update((a.asname or a.name).split(".")[0] for a in node.names)
        elif isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)):
            names.add(node.name)
        elif isinstance(node, ast.Name) and isinstance(node.ctx, (ast.Store, ast.Del)):
            names.add(node.id)
        elif isinstance(node, ast.Global):
            names.update(node.names)
        elif isinstance(node, ast.ExceptHandler) and node.name:
            names.add(node.name)
    return names


def _code_objects(co):
    yield co
    for c in co.co_consts:
        if isinstance(c, types.CodeType):
            yield from _code_objects(c)


_IMPLICIT = set(dir(builtins)) | {"__file__", "__name__", "__doc__", "__spec__", "__path__", "__class__",
                                  "__annotations__", "__qualname__", "__module__"}


def _undefined(src: str, path: str):
    tree = ast.parse(src)
    if any(isinstance(n, ast.ImportFrom) and any(a.name == "*" for a in n.names) for n in ast.walk(tree)):
        return []                                      # names of a star import cannot be listed without importing
    known = _module_names(tree) | _IMPLICIT
    bad = []
    for co in _code_objects(compile(src, path, "exec")):
        for ins in dis.get_instructions(co):
            if ins.opname in ("LOAD_GLOBAL", "LOAD_NAME") and ins.argval not in known:
                line = ins.positions.lineno if ins.positions else "?"
                bad.append(f"{path}:{line}: {ins.argval!r} in {co.co_name}")
    return bad


def test_no_function_loads_an_undefined_global_name():
    probe = "import os\n\ndef f(x):\n    if x:\n        return os.getcwd()\n    return missing_name(x)\n"
    assert _undefined(probe, "probe.py") == ["probe.py:6: 'missing_name' in f"]       # the check sees untaken branches
    bad = []
    for path in _files():
        bad += _undefined(open(path).read(), os.path.relpath(path, ROOT))
    assert not bad, "\n".join(bad)


def test_every_operator_called_from_python_has_a_schema():
    bindings = open(os.path.join(ROOT, "oslo_b200", "csrc", "bindings.cpp")).read()
    schemas = set(re.findall(r'm\.def\(\s*"([A-Za-z0-9_]+)\s*\(', bindings))
    impls = set(re.findall(r'm\.impl\(\s*"([A-Za-z0-9_]+)"', bindings))
    assert impls <= schemas and len(schemas) > 30
    call = re.compile(r'(?:_ext\(\)|load_ext\([^)]*\)|\bext|torch\.ops\.oslo_b200|get_custom_kernels\(\))\.([A-Za-z_][A-Za-z0-9_]*)')
    missing = []
    for path in _files():
        if path.endswith("test_static.py"):
            continue
        for i, line in enumerate(open(path), 1):
            for m in call.finditer(line):
                if m.group(1) not in schemas:
                    missing.append(f"{os.path.relpath(path, ROOT)}:{i}: {m.group(1)}")
    assert not missing, "\n".join(missing)


def _schemas():
    """``{operator: (required positional count, total count, argument names)}`` from the ``m.def`` lines."""
    bindings = open(os.path.join(ROOT, "oslo_b200", "csrc", "bindings.cpp")).read()
    out = {}
    for name, args in re.findall(r'm\.def\(\s*"([A-Za-z0-9_]+)\s*\((.*?)\)\s*->', bindings):
        params = [a.strip() for a in args.split(",") if a.strip()]
        names = [re.sub(r"=.*", "", a).split()[-1] for a in params]
        required = sum(1 for a in params if "=" not in a)
        out[name] = (required, len(params), names)
    return out


def test_operator_calls_pass_as_many_arguments_as_the_schema_takes():
    """Every ``<extension>.<operator>(...)`` call in the tree against the operator's schema: argument count within
    [required, total], keyword names known. (Calls that splat ``*args`` are skipped.)"""
    schemas = _schemas()
    assert schemas["gemm_comm"][1] > 20 and schemas["flash_fwd"][0] == schemas["flash_fwd"][1] - 1
    receiver = re.compile(r"(^_ext\(\)$|load_ext\(.*\)$|^ext$|^torch\.ops\.oslo_b200$|get_custom_kernels\(\)$)")
    bad, seen = [], 0
    for path in _files():
        tree = ast.parse(open(path).read())
        for node in ast.walk(tree):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr in schemas):
                continue
            if not receiver.search(ast.unparse(node.func.value)):
                continue
            if any(isinstance(a, ast.Starred) for a in node.args) or any(k.arg is None for k in node.keywords):
                continue
            seen += 1
            required, total, names = schemas[node.func.attr]
            n = len(node.args) + len(node.keywords)
            unknown = [k.arg for k in node.keywords if k.arg not in names]
            if not (required <= n <= total) or unknown:
                bad.append(f"{os.path.relpath(path, ROOT)}:{node.lineno}: {node.func.attr} takes {required}..{total} "
                           f"arguments, called with {n}" + (f", unknown keywords {unknown}" if unknown else ""))
    assert seen > 40, seen
    assert not bad, "\n".join(bad)


def _signatures(path):
    """``{function: (min positional, max positional or None, keyword names, takes **kwargs)}`` of a module's top level."""
    out = {}
    for node in ast.parse(open(path).read()).body:
        if isinstance(node, ast.FunctionDef):
            a = node.args
            pos = [x.arg for x in a.posonlyargs + a.args]
            required = len(pos) - len(a.defaults)
            kwonly_required = [x.arg for x, d in zip(a.kwonlyargs, a.kw_defaults) if d is None]
            out[node.name] = (required, None if a.vararg else len(pos), set(pos) | {x.arg for x in a.kwonlyargs},
                              a.kwarg is not None, kwonly_required)
    return out


def test_calls_into_the_gpu_only_wrapper_module_match_its_signatures():
    """``ops/cuda_ops.py`` only runs on GPUs, and so do most of its call sites: check every ``cuda_ops.f(...)`` call in
    the tree against ``f``'s signature."""
    sigs = _signatures(os.path.join(ROOT, "oslo_b200", "ops", "cuda_ops.py"))
    bad, seen = [], 0
    for path in _files():
        for node in ast.walk(ast.parse(open(path).read())):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr in sigs
                    and isinstance(node.func.value, ast.Name) and node.func.value.id in ("cuda_ops", "co")):
                continue
            if any(isinstance(a, ast.Starred) for a in node.args) or any(k.arg is None for k in node.keywords):
                continue
            seen += 1
            required, most, names, var_kw, kwonly_required = sigs[node.func.attr]
            given_kw = {k.arg for k in node.keywords}
            n_pos = len(node.args)
            problems = []
            if most is not None and n_pos > most:
                problems.append(f"{n_pos} positional arguments, at most {most}")
            if not var_kw and given_kw - names:
                problems.append(f"unknown keywords {sorted(given_kw - names)}")
            if n_pos + len(given_kw) < required:
                problems.append(f"{n_pos + len(given_kw)} arguments, at least {required}")
            if [k for k in kwonly_required if k not in given_kw]:
                problems.append("missing keyword-only arguments")
            if problems:
                bad.append(f"{os.path.relpath(path, ROOT)}:{node.lineno}: cuda_ops.{node.func.attr}: " + "; ".join(problems))
    assert seen > 40, seen
    assert not bad, "\n".join(bad)


def test_calls_of_the_symmetric_memory_methods_match_their_signatures():
    """The GPU-only methods of ``FusedTP`` / ``SymmetricFlat`` / ``SymmetricWorkspace`` (unique names) by signature."""
    wanted = {"gemm_all_reduce", "gemm_reduce_scatter", "all_gather_gemm", "reduce_scatter_", "all_gather_", "all_reduce_"}
    sigs = {}
    for rel in ("oslo_b200/parallel/fused_tp.py", "oslo_b200/parallel/symmetric.py"):
        for node in ast.walk(ast.parse(open(os.path.join(ROOT, rel)).read())):
            if isinstance(node, ast.ClassDef):
                for f in node.body:
                    if isinstance(f, ast.FunctionDef) and f.name in wanted:
                        pos = [x.arg for x in f.args.args][1:]                      # without self
                        sigs[f.name] = (len(pos) - len(f.args.defaults), len(pos), set(pos) | {x.arg for x in f.args.kwonlyargs})
    assert set(sigs) == wanted, sorted(wanted - set(sigs))
    bad, seen = [], 0
    for path in _files():
        for node in ast.walk(ast.parse(open(path).read())):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr in sigs):
                continue
            if any(isinstance(a, ast.Starred) for a in node.args) or any(k.arg is None for k in node.keywords):
                continue
            seen += 1
            required, most, names = sigs[node.func.attr]
            kw = {k.arg for k in node.keywords}
            n = len(node.args)
            if n > most or kw - names or n + len(kw) < required:
                bad.append(f"{os.path.relpath(path, ROOT)}:{node.lineno}: {node.func.attr} takes {required}..{most}, "
                           f"got {n} positional and keywords {sorted(kw)}")
    assert seen > 15, seen
    assert not bad, "\n".join(bad)


def test_configuration_switches_that_the_code_reads_exist():
    """``get_config().<name>`` anywhere in the tree names a field of ``OsloConfig`` (a misspelt switch in a GPU-only
    branch would only show on a GPU)."""
    cfg_src = ast.parse(open(os.path.join(ROOT, "oslo_b200", "config.py")).read())
    fields = set()
    for node in ast.walk(cfg_src):
        if isinstance(node, ast.ClassDef) and node.name == "OsloConfig":
            fields = {s.target.id for s in node.body if isinstance(s, ast.AnnAssign)} | \
                     {f.name for f in node.body if isinstance(f, ast.FunctionDef)}
    assert "fused_tp_comm" in fields and "pp_reserved_sms" in fields
    bad, seen = [], 0
    for path in _files():
        for node in ast.walk(ast.parse(open(path).read())):
            if (isinstance(node, ast.Attribute) and isinstance(node.value, ast.Call)
                    and isinstance(node.value.func, ast.Name) and node.value.func.id == "get_config"):
                seen += 1
                if node.attr not in fields:
                    bad.append(f"{os.path.relpath(path, ROOT)}:{node.lineno}: get_config().{node.attr}")
    assert seen > 10 and not bad, "\n".join(bad)
