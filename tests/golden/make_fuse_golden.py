"""Extracts the folded #const.Fuse vectors of the reference's lit test into tests/golden/fuse_golden.json.

Source: tests/lit/NPU/dialect/const/passes/constant_folding.mlir of the reference checkout, functions
@FoldSplatFusedConstant, @FoldFusedSignedQuantizedWeightsMixedPrecision and @FoldFusedWeightWithMajorityOfF16Type:
the base constants (dense<...> literals of the weights table and the weights) and the folded result of the
CHECK line. The element types and transformation lists of the three cases are short and are written out in
tests/test_fuse_golden.py next to the lines they come from.

Run where the reference is checked out:
    python tests/golden/make_fuse_golden.py <reference root>
"""
import json
import os
import re
import sys

CASES = ["FoldSplatFusedConstant", "FoldFusedSignedQuantizedWeightsMixedPrecision", "FoldFusedWeightWithMajorityOfF16Type"]
NUM = re.compile(r"-?\d+\.?\d*(?:[eE][-+]?\d+)?")


def numbers(literal):
    return [float(x) if any(c in x for c in ".eE") else int(x) for x in NUM.findall(literal)]


def dense_literals(text):
    """(literal, type string) of every dense<...> : tensor<...> in `text`, in order."""
    out = []
    for m in re.finditer(r"dense<", text):
        i = m.end()
        depth = 0
        j = i
        while True:
            c = text[j]
            if c == "[":
                depth += 1
            elif c == "]":
                depth -= 1
            elif c == ">" and depth == 0:
                break
            j += 1
        ty = re.match(r"\s*:\s*tensor<([^>]*)>", text[j + 1:])
        out.append((text[i:j], ty.group(1) if ty else None))
    return out


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("VPUX_REFERENCE_ROOT", "")
    path = os.path.join(root, "tests", "lit", "NPU", "dialect", "const", "passes", "constant_folding.mlir")
    text = open(path).read()
    blocks = text.split("// -----")
    fixture = {}
    for name in CASES:
        block = next(b for b in blocks if "@" + name + "(" in b)
        line_of = text[:text.index("@" + name + "(")].count("\n") + 1
        body, check = block.split("// CHECK", 1)[0], block[block.index("CHECK-SAME{LITERAL}"):]
        lits = dense_literals(body)
        # Fuse<fusedType, weightsTable=<dense...>, weights=<dense...>, [...]>: the literals after the first (the
        # declared base, which Fuse ignores) are the weights table and the weights
        table_lit, table_ty = lits[1]
        weights_lit, weights_ty = lits[2]
        result_lit, result_ty = dense_literals(check)[0]
        fixture[name] = {
            "line": line_of,
            "weights_table": {"type": table_ty, "values": numbers(table_lit)},
            "weights": {"type": weights_ty, "values": numbers(weights_lit)},
            "result": {"type": result_ty, "values": numbers(result_lit)},
        }
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fuse_golden.json")
    with open(out, "w") as f:
        json.dump(fixture, f, separators=(",", ":"))
    for k, v in fixture.items():
        print(k, "line", v["line"], {p: (v[p]["type"], len(v[p]["values"])) for p in ("weights_table", "weights", "result")})


if __name__ == "__main__":
    main()
