"""Writes tests/golden/engine_client_surface.json: the method names and parameter lists (name,
has-default) of the reference's native Python classes on the save/load path, read from its stub
file python/pegaflow/pegaflow.pyi with `ast` (nothing is imported or executed).

    python tests/golden/gen_client_surface.py <path to the reference checkout>
"""
import ast
import json
import os
import sys

CLASSES = ("EngineRpcClient", "PyLoadState", "QueryReady", "QueryLoading")


def surface(stub_path):
    tree = ast.parse(open(stub_path).read())
    out = {}
    for node in tree.body:
        if not isinstance(node, ast.ClassDef) or node.name not in CLASSES:
            continue
        methods = {}
        for item in node.body:
            if not isinstance(item, ast.FunctionDef):
                continue
            a = item.args
            positional = a.posonlyargs + a.args
            n_defaults = len(a.defaults)
            params = []
            for i, arg in enumerate(positional):
                if arg.arg == "self":
                    continue
                params.append([arg.arg, i >= len(positional) - n_defaults])
            methods[item.name] = params
        fields = [item.target.id for item in node.body if isinstance(item, ast.AnnAssign)]
        out[node.name] = {"methods": methods, "fields": fields}
    return out


if __name__ == "__main__":
    ref = sys.argv[1]
    data = {"source": "python/pegaflow/pegaflow.pyi", "classes": surface(os.path.join(ref, "python/pegaflow/pegaflow.pyi"))}
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "engine_client_surface.json"), "w") as f:
        json.dump(data, f, sort_keys=True)
        f.write("\n")
