"""Import direction of the package, checked on the AST: kernels and containers at the bottom,
the engine above them, serving / training / CLI on top.  A lower layer never imports a higher one.
Counterpart of the reference's tests/test_layering.py."""
import ast
import os

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tilerl_b200")

# level of every top-level module / subpackage; imports may only point to the same or a lower level
LEVEL = {
    "config": 0, "formats": 0, "tokenizer": 0, "ledger": 0, "recipes": 0, "benchrec": 0, "build": 0,
    "ops": 1, "tape": 1, "parallel": 1, "models": 1, "optim": 1,
    "batch": 2, "kv": 2, "kv_tiers": 2, "sparse": 2, "spec": 2, "graph": 2, "memory": 2, "kernel_cost": 2,
    "calibration": 2, "checkpoint": 2, "merge": 2, "mega": 2,
    "sparse_index": 3, "engine": 3,
    "factory": 4, "evals": 4, "server": 4,
    "generate": 5, "rl": 5,
    "cli": 6, "utils": 6, "suites": 6,
}


def _top(parts):
    return parts[1] if len(parts) > 1 else parts[0]


def _edges():
    out = set()
    for dp, _, files in os.walk(ROOT):
        for f in files:
            if not f.endswith(".py"):
                continue
            path = os.path.join(dp, f)
            mod = os.path.relpath(path, os.path.dirname(ROOT))[:-3].split(os.sep)
            if mod[-1] == "__init__":
                mod = mod[:-1]
            if len(mod) < 2:
                continue
            for node in ast.walk(ast.parse(open(path).read())):
                if not isinstance(node, ast.ImportFrom):
                    continue
                if node.level:
                    base = mod[:-node.level] if f != "__init__.py" else mod[:len(mod) - node.level + 1]
                    targets = [base + node.module.split(".")] if node.module else [base + [a.name] for a in node.names]
                elif node.module and node.module.startswith("tilerl_b200."):
                    targets = [node.module.split(".")]
                else:
                    continue
                for t in targets:
                    if len(t) > 1 and _top(t) != _top(mod):
                        out.add((_top(mod), _top(t)))
    return out


def test_every_module_has_a_level():
    names = {f[:-3] for f in os.listdir(ROOT) if f.endswith(".py") and f != "__init__.py"}
    names |= {d for d in os.listdir(ROOT) if os.path.isdir(os.path.join(ROOT, d)) and not d.startswith("_")}
    assert names - set(LEVEL) == set(), names - set(LEVEL)


def test_imports_point_downward():
    bad = sorted((a, b) for a, b in _edges() if a in LEVEL and b in LEVEL and LEVEL[b] > LEVEL[a])
    assert bad == [], bad


def test_serving_layer_sees_only_the_engine():
    assert {b for a, b in _edges() if a == "server"} <= {"engine", "tokenizer", "config"}
