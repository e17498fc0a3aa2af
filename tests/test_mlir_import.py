"""The torch-mlir linalg text -> layer plan importer (CPU): against nncv's own ResNet-18 fixtures when
the nncv tree is at hand, against the committed golden plan otherwise, and on synthetic modules."""
import ctypes
import os

import numpy as np
import pytest

from nncv_b200 import mlir_import as mi
from nncv_b200._lib import lib
import plan_util as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("NNCV_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
HAVE_REF = os.path.isfile(os.path.join(REF, "tests/Nets/Res18.mlir"))


def c_check(text):
    n, k, o = ctypes.c_size_t(), ctypes.c_int(), ctypes.c_int()
    rc = lib().nncv_b200_plan_check(("plan:" + text).encode(), ctypes.byref(n), ctypes.byref(k), ctypes.byref(o))
    return rc, n.value, k.value, o.value


def c_text(net):
    buf = ctypes.create_string_buffer(1 << 16)
    assert lib().nncv_b200_plan_text(net.encode(), buf, len(buf)) > 0
    return buf.value.decode()


def structure(nodes):
    keys = ("kind", "id", "in", "res", "cin", "cout", "k", "stride", "pad", "relu")
    return [tuple(n.get(k) for k in keys) for n in nodes]


def test_builtin_plans_of_library_and_python_agree():
    for d in (18, 50):
        assert c_text(f"resnet{d}") == mi.builtin_plan(d).to_text()


def test_golden_res18_plan_matches_builtin_structure_and_constant_order(golden_dir):
    """The plan read from tests/Nets/Res18.mlir has the built-in plan's nodes one for one.  Its offsets
    differ only because torch-mlir merged equal constants in that (weight-elided) file: three
    batch-norm vectors are shared, 896 elements fewer; the ORDER of the parameters is the built-in one."""
    text = open(os.path.join(golden_dir, "res18_from_mlir.plan")).read()
    total, out, nodes = P.parse_plan_text(text)
    bt, bo, bnodes = P.parse_plan_text(c_text("resnet18"))
    assert out == bo == 1000 and structure(nodes) == structure(bnodes)
    assert bt - total == 896
    roles = [(i, r) for i, n in enumerate(nodes) for r in ("w", "b", "gamma", "beta", "mean", "var") if r in n]
    count = {}
    for i, r in roles:
        count[nodes[i][r]] = count.get(nodes[i][r], 0) + 1
    shared = [(i, r) for i, r in roles if count[nodes[i][r]] > 1]
    # the merged constants: the batch-norm beta of the downsample branch and of the block's second conv
    # (both all-zero in a freshly initialised torchvision model) in the three blocks that change resolution
    assert len(shared) == 6 and all(r == "beta" for _, r in shared)
    assert sum(nodes[i]["cout"] for i, _ in shared) // 2 == 896
    own = [a for a in roles if a not in shared]
    for a in own:
        for b in own:
            if bnodes[a[0]][a[1]] < bnodes[b[0]][b[1]]:
                assert nodes[a[0]][a[1]] < nodes[b[0]][b[1]]
    rc, n, k, o = c_check(text)
    assert (rc, n, k, o) == (0, total, len(nodes), 1000)


@pytest.mark.skipif(not HAVE_REF, reason="needs the nncv source tree")
def test_reference_fixtures_import_to_the_golden_plan(golden_dir):
    gold = open(os.path.join(golden_dir, "res18_from_mlir.plan")).read()
    assert mi.import_mlir_file(os.path.join(REF, "tests/Nets/Res18.mlir")).to_text() == gold
    assert mi.import_mlir_file(os.path.join(REF, "tests/Nets/Res18-half.mlir")).to_text() == gold   # the f16 module
    p = mi.import_mlir_file(os.path.join(REF, "tests/Nets/Res18.mlir"))
    # constants in module order: fc.bias, fc.weight, then groups from the last layer to the first
    assert p.constants[0][1] == (1000,) and p.constants[1][1] == (1000, 512) and p.constants[-1][1] == (64, 3, 7, 7)


@pytest.mark.skipif(not HAVE_REF, reason="needs the nncv source tree")
@pytest.mark.parametrize("name", ["Yolov5s.mlir"])
def test_modules_outside_the_recognised_set_are_refused_with_a_line_number(name):
    with pytest.raises(mi.PlanImportError, match=r"line \d+"):
        mi.import_mlir_file(os.path.join(REF, "tests/Nets", name))


def test_synthetic_module_imports_whatever_the_batchnorm_operand_order():
    a = mi.import_mlir(P.small_net_mlir())
    b = mi.import_mlir(P.small_net_mlir(bn_order=("var", "mean", "gamma", "beta")))
    assert a.to_text() == b.to_text()
    total, out, nodes = P.parse_plan_text(a.to_text())
    assert out == 10 and [n["kind"] for n in nodes] == ["conv", "maxpool", "conv", "conv", "conv", "conv", "conv", "avgpool", "fc"]
    # the projection conv (node 4) runs before the conv that adds its result, although the module lists it later
    assert nodes[4]["res"] == nodes[3]["id"] and nodes[3]["k"] == 1 and nodes[3]["relu"] == 0
    assert nodes[6]["res"] == nodes[5]["id"]          # identity residual
    assert c_check(a.to_text())[0] == 0
    tensors = P.plan_tensors(nodes)
    assert sum(int(__import__("numpy").prod(s)) for _, s, _ in tensors) == total


@pytest.mark.skipif(not HAVE_REF, reason="needs the nncv source tree")
def test_mobilenetv3_fixture_imports_to_the_golden_plan(golden_dir):
    gold = open(os.path.join(golden_dir, "mobilenetv3_from_mlir.plan")).read()
    assert mi.import_mlir_file(os.path.join(REF, "tests/Nets/MobileNetV3.mlir")).to_text() == gold


def test_golden_mobilenetv3_plan(golden_dir):
    """MobileNetV3-small as nncv's fixture spells it: 23 convolutions, 11 depthwise convolutions, 9 squeeze-and-excitation
    blocks, the global average pool and two FC layers; 2.55 M parameters in 210 tensors; batch-norm eps 1e-3."""
    text = open(os.path.join(golden_dir, "mobilenetv3_from_mlir.plan")).read()
    total, out, nodes = P.parse_plan_text(text)
    kinds = [n["kind"] for n in nodes]
    assert (total, out, len(nodes)) == (2554968, 1000, 46)
    assert [kinds.count(k) for k in ("conv", "dwconv", "se", "avgpool", "fc")] == [23, 11, 9, 1, 2]
    tensors = P.plan_tensors(nodes)
    assert len(tensors) == 210 and sum(int(np.prod(s)) for _, s, _ in tensors) == total
    assert abs(P._eps(nodes[0]) - 1e-3) < 1e-9 and nodes[0]["act"] == 3 and nodes[1]["kind"] == "dwconv" and nodes[1]["act"] == 1
    assert sum(1 for n in nodes if n["kind"] == "conv" and n["res"] >= 0) == 6          # the residual blocks of the small variant
    assert nodes[-2]["act"] == 3 and nodes[-2]["cout"] == 1024
    rc, n_params, n_nodes, feats = c_check(text)
    assert (rc, n_params, n_nodes, feats) == (0, total, 46, 1000)
    assert c_text("plan:" + text) == text                                             # the library's parser and printer agree


def test_synthetic_mobile_module():
    text = mi.import_mlir(P.small_mobile_mlir()).to_text()
    total, out, nodes = P.parse_plan_text(text)
    assert [n["kind"] for n in nodes] == ["conv", "dwconv", "se", "conv", "conv", "dwconv", "se", "conv", "conv", "avgpool", "fc", "fc"]
    assert [n.get("act", n.get("relu", 0)) for n in nodes] == [3, 1, 0, 0, 1, 3, 0, 0, 3, 0, 3, 0]
    assert nodes[7]["res"] == nodes[3]["id"] and nodes[2]["cr"] == 8 and nodes[6]["cr"] == 24
    assert c_check(text)[0] == 0 and c_text("plan:" + text) == text
    assert sum(int(np.prod(s)) for _, s, _ in P.plan_tensors(nodes)) == total
    # a second reader of the tensor a squeeze-and-excitation block scales in place is refused by the library
    bad = text.replace("conv id=4 in=3 res=-1 cin=16", "conv id=4 in=2 res=-1 cin=16")
    assert bad != text and c_check(bad)[0] == 1 and b"scaled in place" in lib().nncv_b200_last_error()
    # a hard-swish whose last multiply reads another tensor is not a hard-swish
    src = P.small_mobile_mlir()
    with pytest.raises(mi.PlanImportError):
        mi.import_mlir(src.replace("arith.divf %in, %sixf", "arith.divf %in, %three", 1))


def test_unsupported_patterns_raise():
    good = P.small_net_mlir()
    with pytest.raises(mi.PlanImportError, match="ugt"):
        mi.import_mlir(good.replace("arith.cmpf ugt", "arith.cmpf ogt"))
    with pytest.raises(mi.PlanImportError, match="eps"):
        mi.import_mlir(good.replace("1.000000e-05 : f64", "2.000000e+00 : f64"))
    with pytest.raises(mi.PlanImportError, match="dilated"):
        mi.import_mlir(good.replace("dilations = dense<1>", "dilations = dense<2>", 1))
    with pytest.raises(mi.PlanImportError):
        mi.import_mlir("module {\n}\n")


def test_library_refuses_malformed_plans():
    good = mi.import_mlir(P.small_net_mlir()).to_text()
    assert c_check(good)[0] == 0
    assert c_check(good.replace("nncv_b200_plan 1", "nncv_b200_plan 7"))[0] == 1
    assert c_check(good.replace("in=2 res=-1 cin=16", "in=5 res=-1 cin=16", 1))[0] == 1      # reads a later tensor
    assert c_check(good.replace("cin=64 cout=128 k=1", "cin=32 cout=128 k=1"))[0] == 1          # channel mismatch
    assert c_check(good.replace("params 206330", "params 1000"))[0] == 1                        # offsets past the blob
    assert c_check("\n".join(good.splitlines()[:-1]) + "\n")[0] == 1                            # no FC node
    assert lib().nncv_b200_plan_check(b"/nonexistent/x.plan", None, None, None) == 1
