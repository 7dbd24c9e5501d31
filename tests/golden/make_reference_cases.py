"""Extracts the parameter tuples of the reference's own operator test into a JSON fixture.

    python tests/golden/make_reference_cases.py [path to hustvl/MoDA checkout]

Reads ``libs/moda_triton/tests/ops/test_moda.py`` of the reference (the module-level
``TEST_CASES`` list, tests/ops/test_moda.py:95-198: tuples ``(B, T_kv, H, K, V, L, group,
dtype_name, scale)``) without importing it, and writes ``reference_test_cases.json`` beside this
script.  ``tests/test_reference_cases_gpu.py`` runs every tuple through this library against the
CPU oracle with the reference test's seed (2025).  The reference is only needed to regenerate
the fixture, never to run the tests.
"""
import ast
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MODA_REFERENCE_DIR", os.path.join(os.sep, "root", "reference"))
    path = os.path.join(ref, "libs", "moda_triton", "tests", "ops", "test_moda.py")
    tree = ast.parse(open(path).read())
    cases = None
    for node in tree.body:
        if isinstance(node, ast.Assign) and any(getattr(t, "id", None) == "TEST_CASES" for t in node.targets):
            cases = ast.literal_eval(node.value)
    assert cases, "TEST_CASES not found"
    out = {"source": "libs/moda_triton/tests/ops/test_moda.py: TEST_CASES", "seed": 2025,
           "fields": ["B", "T_kv", "H", "K", "V", "L", "group", "dtype_name", "scale"],
           "cases": [list(c) for c in cases]}
    with open(os.path.join(HERE, "reference_test_cases.json"), "w") as f:
        f.write('{"source": %s, "seed": %d,\n "fields": %s,\n "cases": [\n'
                % (json.dumps(out["source"]), out["seed"], json.dumps(out["fields"])))
        f.write(",\n".join("  " + json.dumps(c) for c in out["cases"]))
        f.write("\n ]}\n")
    print(len(cases), "cases")


if __name__ == "__main__":
    main()
