"""torch-mlir "linalg-on-tensors" text -> layer plan for libnncv_b200.so.

nncv compiles such a module (tests/Nets/Res18.mlir is its ResNet-18 fixture) op by op; its
`-split-params` pass moves every tensor constant into one blob and addresses constant i at the
element offset sum(numel of the constants before it), in module walk order
(src/nncv/compiler/Conversion/Transforms/SplitParamsFlatArray.cpp:48-56, 84-92, 109-114).  This
importer does the part of that job the runtime needs: it reads the `@forward` function, recognises

    tensor.pad(0) -> linalg.conv_2d_nchw_fchw -> batch-norm generic [-> add generic] [-> ReLU generic]
    tensor.pad(-inf) -> linalg.pooling_nchw_max
    linalg.pooling_nchw_sum over the whole map -> divf generic           (global average pool)
    tensor.collapse_shape -> transpose generic -> linalg.matmul -> bias add generic   (FC)

(op shapes as in Res18.mlir:118-629) and writes the plan text `nncv_b200_load` accepts in place of
a built-in network name.  The elementwise generics are classified by their bodies, not by position:
batch-norm operand roles come from the dataflow of the region (the value added to eps under the
rsqrt is the variance, the one subtracted from the input is the mean, ...), so a different operand
order in another export still imports correctly.  Anything outside these patterns raises
PlanImportError naming the line.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


class PlanImportError(ValueError):
    pass


@dataclass
class Node:
    kind: str                      # conv | maxpool | avgpool | fc
    order: int                     # creation order in the module
    inp: object = None             # producing Node, or 0 for the network input
    res: Optional["Node"] = None
    cin: int = 0
    cout: int = 0
    k: int = 1
    stride: int = 1
    pad: int = 0
    relu: int = 0
    w: int = -1
    b: int = -1
    gamma: int = -1
    beta: int = -1
    mean: int = -1
    var: int = -1
    id: int = 0

    def fields(self) -> Dict[str, int]:
        in_id = 0 if self.inp == 0 else self.inp.id
        if self.kind == "conv":
            d = dict(id=self.id, **{"in": in_id}, res=self.res.id if self.res else -1, cin=self.cin, cout=self.cout,
                     k=self.k, stride=self.stride, pad=self.pad, relu=self.relu, w=self.w)
            if self.gamma >= 0:
                d.update(gamma=self.gamma, beta=self.beta, mean=self.mean, var=self.var)
            return d
        if self.kind == "maxpool":
            return dict(id=self.id, **{"in": in_id}, k=self.k, stride=self.stride, pad=self.pad)
        if self.kind == "avgpool":
            return dict(id=self.id, **{"in": in_id})
        return dict(id=self.id, **{"in": in_id}, cin=self.cin, cout=self.cout, w=self.w, b=self.b)


@dataclass
class Plan:
    nodes: List[Node] = field(default_factory=list)
    total: int = 0
    out_features: int = 0
    constants: List[Tuple[str, Tuple[int, ...], int]] = field(default_factory=list)   # (ssa name, shape, element offset)

    def to_text(self) -> str:
        lines = ["nncv_b200_plan 1", f"params {self.total} out {self.out_features}"]
        for n in self.nodes:
            lines.append(n.kind + " " + " ".join(f"{k}={v}" for k, v in n.fields().items()))
        return "\n".join(lines) + "\n"

    def write(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.to_text())

    def signature(self):
        """Node tuples for comparing two plans."""
        return [(n.kind, tuple(sorted(n.fields().items()))) for n in self.nodes]


# ------------------------------------------------------------------------------ parsing
_TENSOR = re.compile(r"tensor<((?:\d+x)*)(f32|f16|bf16|f64|i64|i1)>")
_STMT = re.compile(r"^\s*(%[\w.]+)(?::\d+)?\s*=\s*([\w.]+)\b(.*)$")


def _shape(type_text: str) -> Tuple[int, ...]:
    m = _TENSOR.search(type_text)
    if not m:
        raise PlanImportError(f"no tensor type in {type_text!r}")
    return tuple(int(v) for v in m.group(1).split("x") if v)


def _split_top(text: str) -> List[str]:
    """Split at commas that are not inside <>, [] or ()."""
    out, depth, cur = [], 0, ""
    for ch in text:
        if ch in "<[(":
            depth += 1
        elif ch in ">])":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur.strip())
    return out


def _operands(text: str, key: str) -> Tuple[List[str], List[str]]:
    """`key(%a, %b : t1, t2)` -> ([%a, %b], [t1, t2])."""
    i = text.find(key + "(")
    if i < 0:
        return [], []
    j, depth = i + len(key) + 1, 1
    start = j
    while depth:
        if text[j] == "(":
            depth += 1
        elif text[j] == ")":
            depth -= 1
        j += 1
    inner = text[start:j - 1]
    names, _, types = inner.partition(" : ")
    return [n.strip() for n in names.split(",") if n.strip()], _split_top(types)


@dataclass
class Stmt:
    line: int
    result: str
    op: str
    head: str          # text after the op name on the first line
    body: List[str]    # region lines (without the block-argument line)
    block_args: List[str]
    tail: str          # text of the closing line of a region op


def _statements(text: str) -> List[Stmt]:
    lines = text.splitlines()
    out: List[Stmt] = []
    i = 0
    in_func = False
    while i < len(lines):
        ln = lines[i]
        if "func.func @forward" in ln:
            in_func = True
            m = re.search(r"\(([^)]*)\)", ln)
            out.append(Stmt(i + 1, "%arg0", "func.arg", m.group(1) if m else "", [], [], ""))
            i += 1
            continue
        if not in_func:
            i += 1
            continue
        s = ln.strip()
        if s.startswith("return"):
            out.append(Stmt(i + 1, "", "return", s[len("return"):].strip(), [], [], ""))
            break
        m = _STMT.match(ln)
        if not m:
            i += 1
            continue
        res, op, head = m.group(1), m.group(2), m.group(3)
        body, args, tail = [], [], ""
        if head.rstrip().endswith("{"):
            i += 1
            while i < len(lines) and not lines[i].strip().startswith("}"):
                b = lines[i].strip()
                if b.startswith("^"):
                    args = re.findall(r"(%[\w.]+)\s*:", b)
                else:
                    body.append(b)
                i += 1
            tail = lines[i].strip() if i < len(lines) else ""
        out.append(Stmt(i + 1, res, op, head, body, args, tail))
        i += 1
    if not in_func:
        raise PlanImportError("the module has no func.func @forward")
    return out


def _body_ops(st: Stmt) -> List[Tuple[str, str, List[str]]]:
    """Region statements as (result, op, operand names)."""
    ops = []
    for b in st.body:
        m = _STMT.match(b)
        if m:
            rest = m.group(3).split(":")[0]
            ops.append((m.group(1), m.group(2), re.findall(r"%[\w.]+", rest)))
        elif b.startswith("linalg.yield"):
            ops.append(("", "linalg.yield", re.findall(r"%[\w.]+", b)))
    return ops


# ------------------------------------------------------------------------------ recognition
def _scalar_value(text: str) -> Optional[float]:
    """Value of a scalar arith.constant (`0.000000e+00 : f32`, `0xFF800000 : f32`, `1.0e-05 : f64`)."""
    m = re.match(r"\s*(\S+)\s*:\s*(f32|f16|f64)", text)
    if not m:
        return None
    v = m.group(1)
    if v.lower().startswith("0x"):
        import struct
        bits = int(v, 16)
        if m.group(2) == "f32":
            return struct.unpack("<f", struct.pack("<I", bits))[0]
        if m.group(2) == "f16":
            return float(struct.unpack("<e", struct.pack("<H", bits))[0])
        return struct.unpack("<d", struct.pack("<Q", bits))[0]
    try:
        return float(v)
    except ValueError:
        return None


def import_mlir(text: str) -> Plan:
    """Plan of the `@forward` function of a torch-mlir linalg-on-tensors module."""
    stmts = _statements(text)
    plan = Plan()
    consts: Dict[str, Tuple[Tuple[int, ...], int]] = {}    # tensor constants: name -> (shape, element offset)
    scalars: Dict[str, float] = {}
    val: Dict[str, tuple] = {}         # SSA name -> symbolic value
    shapes: Dict[str, Tuple[int, ...]] = {}
    uses: Dict[str, int] = {}
    nodes: List[Node] = []
    offset = 0

    for st in stmts:   # use counts first: a fused intermediate must have exactly one reader
        if st.op == "func.arg":
            continue
        text = re.sub(r"outs\([^)]*\)", "", st.head + " " + st.tail)   # an `outs` operand is the destination, not a reader
        for n in re.findall(r"%[\w.]+", text):
            uses[n] = uses.get(n, 0) + 1

    def err(st: Stmt, msg: str):
        raise PlanImportError(f"line {st.line}: {msg}")

    def new_node(kind: str, **kw) -> Node:
        n = Node(kind=kind, order=len(nodes), **kw)
        nodes.append(n)
        return n

    def tensor_of(st: Stmt, name: str):
        """The materialised tensor a consumer reads: the network input or a finished node."""
        v = val.get(name)
        if v is None:
            err(st, f"{name} is not a value this importer tracks")
        if v[0] == "input":
            return 0
        if v[0] == "node":
            return v[1]
        err(st, f"{name} ({v[0]}) cannot be read as a tensor here")

    def single_use(st: Stmt, name: str):
        if uses.get(name, 0) != 1:
            err(st, f"{name} is fused into its consumer but has {uses.get(name, 0)} readers")

    for st in stmts:
        if st.op == "func.arg":
            shp = _shape(st.head)
            if len(shp) != 4 or shp[1] != 3:
                err(st, f"the input must be [N,3,H,W], got {shp}")
            val["%arg0"] = ("input",)
            shapes["%arg0"] = shp
        elif st.op == "arith.constant":
            if "tensor<" in st.head:
                shp = _shape(st.head)
                consts[st.result] = (shp, offset)
                plan.constants.append((st.result, shp, offset))
                offset += int(math.prod(shp)) if shp else 1
                val[st.result] = ("const", st.result)
                shapes[st.result] = shp
            else:
                v = _scalar_value(st.head)
                if v is not None:
                    scalars[st.result] = v
        elif st.op in ("tensor.empty", "linalg.fill", "arith.cmpi", "cf.assert"):
            continue
        elif st.op == "tensor.pad":
            src = re.match(r"\s*(%[\w.]+)", st.head).group(1)
            lo = [int(v) for v in re.search(r"low\[([^\]]*)\]", st.head).group(1).split(",")]
            hi = [int(v) for v in re.search(r"high\[([^\]]*)\]", st.head).group(1).split(",")]
            y = [b for b in st.body if b.startswith("tensor.yield")]
            fill = scalars.get(re.findall(r"%[\w.]+", y[0])[0]) if y else None
            if lo != hi or lo[0] or lo[1] or lo[2] != lo[3] or fill is None:
                err(st, "only symmetric spatial padding with a constant is supported")
            val[st.result] = ("padded", src, lo[2], fill)
            shapes[st.result] = _shape(st.tail.split(" to ")[-1])
        elif st.op == "linalg.conv_2d_nchw_fchw":
            ins, types = _operands(st.head, "ins")
            stride = int(re.search(r"strides = dense<(\d+)>", st.head).group(1))
            if int(re.search(r"dilations = dense<(\d+)>", st.head).group(1)) != 1:
                err(st, "dilated convolutions are not supported")
            src, pad = ins[0], 0
            v = val.get(src)
            if v and v[0] == "padded":
                if v[3] != 0.0:
                    err(st, "a convolution input must be padded with zeros")
                single_use(st, src)
                src, pad = v[1], v[2]
            if ins[1] not in consts:
                err(st, "the filter must be a constant")
            k, c, r, s = consts[ins[1]][0]
            if r != s:
                err(st, "only square filters are supported")
            n = new_node("conv", inp=tensor_of(st, src), cin=c, cout=k, k=r, stride=stride, pad=pad, w=consts[ins[1]][1])
            val[st.result] = ("conv", n, "raw")
            shapes[st.result] = _shape(st.head.split("->")[-1])
        elif st.op == "linalg.generic":
            ins, types = _operands(st.head, "ins")
            ops = _body_ops(st)
            kinds = [o[1] for o in ops]
            shapes[st.result] = _shape(st.tail.split("->")[-1])
            arg = dict(zip(st.block_args, ins))   # block argument -> outer operand
            if "math.rsqrt" in kinds:
                # batch-norm: roles from the dataflow of the region
                d = {o[0]: o for o in ops}
                rs = next(o for o in ops if o[1] == "math.rsqrt")
                addv = d[rs[2][0]]
                var_arg = next(a for a in addv[2] if a in arg)
                eps_src = next(a for a in addv[2] if a not in arg)
                eps = scalars.get(d[eps_src][2][0]) if eps_src in d else scalars.get(eps_src)
                sub = next(o for o in ops if o[1] == "arith.subf")
                x_arg, mean_arg = sub[2][0], sub[2][1]
                mul1 = next(o for o in ops if o[1] == "arith.mulf" and sub[0] in o[2] and rs[0] in o[2])
                mul2 = next(o for o in ops if o[1] == "arith.mulf" and mul1[0] in o[2])
                gamma_arg = next(a for a in mul2[2] if a in arg)
                add2 = next(o for o in ops if o[1] == "arith.addf" and mul2[0] in o[2])
                beta_arg = next(a for a in add2[2] if a in arg)
                if eps is None or abs(eps - 1e-5) > 1e-12:
                    err(st, f"batch-norm eps {eps} is not 1e-5")
                v = val.get(arg[x_arg])
                if not v or v[0] != "conv" or v[2] != "raw":
                    err(st, "batch-norm must follow a convolution directly")
                single_use(st, arg[x_arg])
                n = v[1]
                for role, a in (("gamma", gamma_arg), ("beta", beta_arg), ("mean", mean_arg), ("var", var_arg)):
                    if arg[a] not in consts or consts[arg[a]][0] != (n.cout,):
                        err(st, f"batch-norm {role} must be a constant of {n.cout} values")
                    setattr(n, role, consts[arg[a]][1])
                val[st.result] = ("conv", n, "bn")
            elif "arith.cmpf" in kinds and "arith.select" in kinds:
                cmp_ = next(o for o in ops if o[1] == "arith.cmpf")
                zero = [a for a in cmp_[2] if a not in arg]
                if "ugt" not in " ".join(st.body) or not zero or scalars.get(zero[0]) != 0.0:
                    err(st, "only ReLU written as cmpf ugt x, 0 + select is recognised")
                v = val.get(ins[0])
                if not v or v[0] != "conv" or v[1].relu:
                    err(st, "ReLU must follow a convolution's batch-norm or residual add")
                single_use(st, ins[0])
                v[1].relu = 1
                val[st.result] = ("node", v[1])
            elif kinds == ["arith.addf", "linalg.yield"] and len(ins) == 2 and len(shapes.get(ins[1], ())) == 4:
                # residual add: the operand that is an unfinished conv takes the other one in its epilogue
                a, b = val.get(ins[0]), val.get(ins[1])
                main, other = (ins[0], ins[1]) if a and a[0] == "conv" and not a[1].relu and a[1].res is None else (ins[1], ins[0])
                mv = val.get(main)
                if not mv or mv[0] != "conv" or mv[1].relu or mv[1].res is not None:
                    err(st, "a residual add needs one operand that is a convolution + batch-norm without ReLU")
                single_use(st, main)
                ov = val.get(other)
                if ov and ov[0] == "conv":      # the other branch ends without ReLU (downsample conv + batch-norm)
                    single_use(st, other)
                    val[other] = ("node", ov[1])
                mv[1].res = tensor_of(st, other)
                if mv[1].res == 0:
                    err(st, "the network input cannot be a residual")
                val[st.result] = ("conv", mv[1], "add")
            elif kinds == ["arith.divf", "linalg.yield"]:
                v = val.get(ins[0])
                div = [a for a in ops[0][2] if a not in arg]
                if not v or v[0] != "sumpool" or not div or scalars.get(div[0]) != float(v[2]):
                    err(st, "divf is only recognised after a sum-pool over the whole map, dividing by its size")
                single_use(st, ins[0])
                val[st.result] = ("node", new_node("avgpool", inp=v[1]))
            elif kinds == ["linalg.yield"] and len(ins) == 1 and ins[0] in consts and len(consts[ins[0]][0]) == 2:
                val[st.result] = ("const_t", ins[0])     # FC weight transposed at run time (Res18.mlir:617-620)
            elif kinds == ["arith.addf", "linalg.yield"] and len(ins) == 2:
                v = val.get(ins[0])
                if not v or v[0] != "fc" or ins[1] not in consts or consts[ins[1]][0] != (v[1].cout,):
                    err(st, "a vector add is only recognised as the bias of the FC layer")
                single_use(st, ins[0])
                v[1].b = consts[ins[1]][1]
                val[st.result] = ("node", v[1])
            else:
                err(st, f"unrecognised linalg.generic body {kinds}")
        elif st.op == "linalg.pooling_nchw_max":
            ins, types = _operands(st.head, "ins")
            stride = int(re.search(r"strides = dense<(\d+)>", st.head).group(1))
            win = _shape(types[1])
            v = val.get(ins[0])
            src, pad = ins[0], 0
            if v and v[0] == "padded":
                if not math.isinf(v[3]) or v[3] > 0:
                    err(st, "a max-pool input must be padded with -inf")
                single_use(st, ins[0])
                src, pad = v[1], v[2]
            if win[0] != win[1]:
                err(st, "only square pooling windows are supported")
            val[st.result] = ("node", new_node("maxpool", inp=tensor_of(st, src), k=win[0], stride=stride, pad=pad))
            shapes[st.result] = _shape(st.head.split("->")[-1])
        elif st.op == "linalg.pooling_nchw_sum":
            ins, types = _operands(st.head, "ins")
            win, shp = _shape(types[1]), _shape(types[0])
            if tuple(win) != tuple(shp[2:]):
                err(st, "only a sum-pool over the whole map (global average pool) is supported")
            val[st.result] = ("sumpool", tensor_of(st, ins[0]), win[0] * win[1])
        elif st.op == "tensor.collapse_shape":
            src = re.match(r"\s*(%[\w.]+)", st.head).group(1)
            val[st.result] = val[src]
        elif st.op == "linalg.matmul":
            ins, types = _operands(st.head, "ins")
            wv = val.get(ins[1])
            if not wv or wv[0] != "const_t":
                err(st, "matmul is only recognised as the FC layer: activations x transposed constant")
            (o, i_), woff = consts[wv[1]]
            x = tensor_of(st, ins[0])
            if x == 0 or x.kind != "avgpool":
                err(st, "the FC layer must read the global average pool")
            n = new_node("fc", inp=x, cin=i_, cout=o, w=woff)
            val[st.result] = ("fc", n)
        elif st.op == "return":
            name = re.findall(r"%[\w.]+", st.head)[0]
            v = val.get(name)
            if not v or v[0] != "node" or v[1].kind != "fc" or v[1].b < 0:
                err(st, "the function must return the FC layer's output")
            plan.out_features = v[1].cout
        elif st.op.startswith("arith.") or st.op.startswith("math."):
            continue
        else:
            err(st, f"unsupported op {st.op}")

    for n in nodes:
        if n.kind == "conv" and n.gamma < 0:
            raise PlanImportError(f"convolution #{n.order} has no batch-norm; plain convolutions are not in the recognised set")
    # forward order: a node runs after the producers of its input and of its residual; otherwise module order
    done, order = set(), []

    def visit(n: Node):
        if id(n) in done:
            return
        for d in (n.inp, n.res):
            if isinstance(d, Node):
                visit(d)
        done.add(id(n))
        order.append(n)

    for n in nodes:
        visit(n)
    for i, n in enumerate(order):
        n.id = i + 1
    plan.nodes = order
    plan.total = offset
    return plan


def import_mlir_file(path: str) -> Plan:
    with open(path) as f:
        return import_mlir(f.read())


def builtin_plan(depth: int) -> Plan:
    """The plan libnncv_b200.so builds for "resnet18" / "resnet50", from the layer tables."""
    from .netspec import conv_groups, fc_in, tensor_order
    off, pos = {}, 0
    for name, shape in tensor_order(depth):
        off[name] = pos
        pos += int(math.prod(shape))
    groups = {g.name: g for g in conv_groups(depth)}
    nodes: List[Node] = []

    def conv(name, inp, res, relu):
        g = groups[name]
        n = Node("conv", len(nodes), inp=inp, res=res, cin=g.cin, cout=g.cout, k=g.k, stride=g.stride, pad=g.pad, relu=relu,
                 w=off[f"{g.name}.weight"], gamma=off[f"{g.bn}.weight"], beta=off[f"{g.bn}.bias"],
                 mean=off[f"{g.bn}.running_mean"], var=off[f"{g.bn}.running_var"])
        nodes.append(n)
        return n

    x = conv("conv1", 0, None, 1)
    x = Node("maxpool", len(nodes), inp=x, k=3, stride=2, pad=1)
    nodes.append(x)
    for l, nb in enumerate((2, 2, 2, 2) if depth == 18 else (3, 4, 6, 3)):
        for b in range(nb):
            p = f"layer{l + 1}.{b}"
            t = conv(f"{p}.conv1", x, None, 1)
            if depth == 50:
                t = conv(f"{p}.conv2", t, None, 1)
            idn = conv(f"{p}.downsample.0", x, None, 0) if f"{p}.downsample.0" in groups else x
            x = conv(f"{p}.conv2" if depth == 18 else f"{p}.conv3", t, idn, 1)
    a = Node("avgpool", len(nodes), inp=x)
    nodes.append(a)
    nodes.append(Node("fc", len(nodes), inp=a, cin=fc_in(depth), cout=1000, w=off["fc.weight"], b=off["fc.bias"]))
    for i, n in enumerate(nodes):
        n.id = i + 1
    return Plan(nodes=nodes, total=pos, out_features=1000)


if __name__ == "__main__":
    import sys
    if len(sys.argv) != 3:
        raise SystemExit("usage: python -m nncv_b200.mlir_import <module.mlir> <out.plan>")
    import_mlir_file(sys.argv[1]).write(sys.argv[2])
