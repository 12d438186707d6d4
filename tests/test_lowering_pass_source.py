"""The MLIR lowering pass (mlir/ConvertNovaContractionsToB200Calls.cpp) cannot be compiled here (no MLIR
toolchain), so what CAN be checked is checked: the call table in its header comment names only functions the
library exports, with the arity the pass passes; the enumerator values it hard-codes are the header's; and every
contraction the textual front-end plans for the reference's pipeline-test fixtures is one of the (init, act)
combinations the pass declares — the two implementations of the same fusion decisions agree."""
import glob
import os
import re

from nova_compiler_b200 import _lib as L
from nova_compiler_b200.frontend import Module

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = open(os.path.join(ROOT, "mlir", "ConvertNovaContractionsToB200Calls.cpp")).read()
HDR = open(os.path.join(ROOT, "include", "nova_b200.h")).read()


def _enum_values(name):
    body = re.search(r"typedef enum %s \{(.*?)\}" % name, HDR, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    return {k: int(v) for k, v in re.findall(r"(NOVA_B200_\w+)\s*=\s*(\d+)", body)}


def test_call_table_names_exported_functions_with_the_right_arity(lib):
    rows = re.findall(r"// @call (.*?)\|\s*(\w+)\s*\|\s*(.*?)\|\s*(.*)", SRC)
    assert len(rows) >= 8
    inits, acts = _enum_values("nova_b200_acc_init"), _enum_values("nova_b200_act")
    for form, callee, init, act in rows:
        assert hasattr(lib, callee) and callee in L.PROTOTYPES, callee
        for token, table in ((init.strip(), inits), (act.strip(), acts)):
            assert token.startswith("(as matched)") or token in table, token
    for callee, n in re.findall(r"// @arity (\w+) (\d+)", SRC):
        assert len(L.PROTOTYPES[callee][1]) == int(n)
    # the pass builds exactly that many call operands: 17 i64, 7 i32, 1 i64
    assert "SmallVector<Type> args(17, i64)" in SRC and "args.append(7, i32)" in SRC


def test_hard_coded_enumerators_match_the_header():
    inits, acts, dts = _enum_values("nova_b200_acc_init"), _enum_values("nova_b200_act"), _enum_values("nova_b200_dtype")
    consts = {k: int(v) for k, v in re.findall(r"\b(k[A-Z]\w+) = (\d+)", SRC)}
    assert consts["kF32"] == dts["NOVA_B200_F32"] and consts["kF16"] == dts["NOVA_B200_F16"] and consts["kBF16"] == dts["NOVA_B200_BF16"]
    assert consts["kActNone"] == acts["NOVA_B200_ACT_NONE"] and consts["kActRelu"] == acts["NOVA_B200_ACT_RELU"]
    assert consts["kActGeluTanh"] == acts["NOVA_B200_ACT_GELU_TANH"]
    assert consts["kInitZero"] == inits["NOVA_B200_INIT_ZERO"] and consts["kInitBiasRow"] == inits["NOVA_B200_INIT_BIAS_ROW"]
    assert consts["kInitResidualFull"] == inits["NOVA_B200_INIT_RESIDUAL_FULL"]
    assert consts["kInitFromC"] == inits["NOVA_B200_INIT_FROM_C"]
    assert consts["kInitBiasAndResidual"] == inits["NOVA_B200_INIT_BIAS_AND_RESIDUAL"]


def test_front_end_plans_of_the_pipeline_fixtures_use_only_declared_combinations():
    declared_init = {"zero", "bias_row", "residual", "bias_row+residual"}
    declared_act = {"none", "relu", "gelu_tanh"}
    seen = set()
    for f in sorted(glob.glob(os.path.join(ROOT, "tests", "golden", "ref_fixtures", "test__pipeline-tests__*.mlir"))):
        text = open(f).read()
        m = Module(text)
        for fn in re.findall(r"func\.func\s+@([\w$.-]+)", re.sub(r"//[^\n]*", "", text)):
            for line in m.plan(fn).splitlines():
                line = line.strip()
                if not line.startswith("gemm "):
                    continue
                init = re.sub(r"\(%[^)]*\)", "", re.search(r"init=(\S+)", line).group(1))
                act = re.search(r"act=(\w+)", line).group(1)
                assert init in declared_init and act in declared_act, (f, line)
                seen.add((init, act))
    # the fixtures exercise the plain, residual, bias+residual and ReLU forms
    assert {("zero", "none"), ("residual", "none"), ("residual", "relu"), ("bias_row+residual", "relu")} <= seen
