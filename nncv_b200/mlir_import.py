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

(op shapes as in Res18.mlir:118-629), and of the MobileNetV3 fixture (tests/Nets/MobileNetV3.mlir)

    tensor.pad(0) -> linalg.depthwise_conv_2d_nchw_chw (collapsed filter) -> batch-norm generic   (:301-319)
    hard-swish  x * min(max(x + 3, 0), 6) / 6  and hard-sigmoid  max(min((x + 3) / 6, 1), 0), each spread
        over four to six single-op generics                                               (:263-295, :345-383)
    squeeze-and-excitation: global average pool -> 1x1 conv + bias -> ReLU -> 1x1 conv + bias ->
        hard-sigmoid -> broadcast multiply                                                   (:319-389)
    residual add without an activation, FC + hard-swish -> FC                                (:1784-1864)

and writes the plan text `nncv_b200_load` accepts in place of
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


def _f32_bits(v: float) -> int:
    """The value rounded to fp32, as its bit pattern (plan fields are integers)."""
    import struct
    return struct.unpack("<I", struct.pack("<f", v))[0]


@dataclass
class Node:
    kind: str                      # conv | dwconv | se | maxpool | avgpool | fc
    order: int                     # creation order in the module
    inp: object = None             # producing Node, or 0 for the network input
    res: Optional["Node"] = None
    cin: int = 0
    cout: int = 0
    k: int = 1
    stride: int = 1
    pad: int = 0
    relu: int = 0
    act: int = 0                   # 0 none, 1 ReLU, 2 hard-sigmoid, 3 hard-swish (the C ABI's activation codes)
    eps: float = 1e-5              # batch-norm epsilon (the f64 constant the module truncates to f32)
    cr: int = 0                    # se: squeezed width
    w2: int = -1                   # se: second 1x1 conv
    b2: int = -1
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
            if self.act > 1:
                d.update(act=self.act)
            if self.gamma >= 0:
                d.update(gamma=self.gamma, beta=self.beta, mean=self.mean, var=self.var)
                if abs(self.eps - 1e-5) > 1e-12:
                    d.update(eps_bits=_f32_bits(self.eps))
            if self.b >= 0:
                d.update(b=self.b)
            return d
        if self.kind == "dwconv":
            d = dict(id=self.id, **{"in": in_id}, c=self.cout, k=self.k, stride=self.stride, pad=self.pad, act=self.act,
                     w=self.w, gamma=self.gamma, beta=self.beta, mean=self.mean, var=self.var)
            if abs(self.eps - 1e-5) > 1e-12:
                d.update(eps_bits=_f32_bits(self.eps))
            return d
        if self.kind == "se":
            return dict(id=self.id, **{"in": in_id}, c=self.cout, cr=self.cr, w1=self.w, b1=self.b, w2=self.w2, b2=self.b2)
        if self.kind == "maxpool":
            return dict(id=self.id, **{"in": in_id}, k=self.k, stride=self.stride, pad=self.pad)
        if self.kind == "avgpool":
            return dict(id=self.id, **{"in": in_id})
        d = dict(id=self.id, **{"in": in_id}, cin=self.cin, cout=self.cout, w=self.w, b=self.b)
        if self.act:
            d.update(act=self.act)
        return d


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
        mi = re.match(r"\s*(-?\d+)\s*:\s*i(64|32)", text)
        return float(mi.group(1)) if mi else None
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
    scalar_tensors: Dict[str, float] = {}
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
        """The materialised tensor a consumer reads: the network input or a finished node.  A convolution
        whose batch-norm (or bias, or residual add) is done and that no activation follows ends here."""
        v = val.get(name)
        if v is None:
            err(st, f"{name} is not a value this importer tracks")
        if v[0] == "input":
            return 0
        if v[0] == "conv" and v[2] in ("bn", "add", "bias"):
            val[name] = v = ("node", v[1])
        if v[0] == "node":
            return v[1]
        err(st, f"{name} ({v[0]}) cannot be read as a tensor here")

    def single_use(st: Stmt, name: str):
        if uses.get(name, 0) != 1:
            err(st, f"{name} is fused into its consumer but has {uses.get(name, 0)} readers")

    # ---- elementwise generics: each is evaluated symbolically over its tensor operands; chains of
    # single-op generics (hard-swish takes five) grow one expression until it matches a known function.
    X = ("x",)
    RELU = ("max", X, 0.0)
    HSWISH = ("mul", ("div", ("min", ("max", ("add", X, 3.0), 0.0), 6.0), 6.0), X)
    HSIGMOID = ("max", ("min", ("div", ("add", X, 3.0), 6.0), 1.0), 0.0)

    def subexprs(e, acc):
        if isinstance(e, tuple) and e != X:
            acc.add(e)
            for c in e[1:]:
                subexprs(c, acc)
        return acc

    PREFIXES = subexprs(HSWISH, set()) | subexprs(HSIGMOID, set())

    def leaves(e, acc):
        if isinstance(e, tuple):
            if e[0] == "t":
                acc.append(e[1])
            else:
                for c in e[1:]:
                    leaves(c, acc)
        return acc

    def subst(e, name):
        """The expression with tensor `name` replaced by the placeholder X."""
        if isinstance(e, tuple):
            if e == ("t", name):
                return X
            return (e[0],) + tuple(subst(c, name) for c in e[1:])
        return e

    def commute(e):
        """Binary ops with the tensor expression first, the constant second; `mul` of two tensors ordered by size."""
        if not isinstance(e, tuple) or e[0] in ("t", "x"):
            return e
        c = [commute(v) for v in e[1:]]
        if e[0] in ("add", "mul", "min", "max") and len(c) == 2:
            if isinstance(c[0], float) and not isinstance(c[1], float):
                c = [c[1], c[0]]
            elif e[0] == "mul" and isinstance(c[0], tuple) and isinstance(c[1], tuple) and len(repr(c[0])) < len(repr(c[1])):
                c = [c[1], c[0]]
        return (e[0],) + tuple(c)

    def body_expr(st: Stmt, ops, arg):
        env = {}
        for ba, outer in arg.items():
            if outer in scalar_tensors:
                env[ba] = float(scalar_tensors[outer])
            else:
                v = val.get(outer)
                env[ba] = v[1] if v and v[0] == "ew" else ("t", outer)

        def get(name):
            if name in env:
                return env[name]
            if name in scalars:
                return float(scalars[name])
            err(st, f"{name} in an elementwise body is neither an operand nor a scalar constant")

        out = None
        for res, op, operands in ops:
            if op == "linalg.yield":
                out = get(operands[0])
            elif op in ("arith.addf", "arith.mulf", "arith.divf", "arith.subf"):
                env[res] = (op[6:9], get(operands[0]), get(operands[1]))
            elif op == "arith.cmpf":
                pred = next((p_ for p_ in ("ugt", "ogt", "olt", "ult") if re.search(r"\b" + p_ + r"\b", " ".join(st.body))), None)
                if pred is None:
                    err(st, "unsupported comparison in an elementwise body")
                env[res] = ("cmp", pred, get(operands[0]), get(operands[1]))
            elif op == "arith.select":
                c, a_, b_ = get(operands[0]), get(operands[1]), get(operands[2])
                if not (isinstance(c, tuple) and c[0] == "cmp" and c[2] == a_ and c[3] == b_):
                    err(st, "select is only recognised as select(cmp(a, b), a, b)")
                # the spellings whose NaN behaviour the kernels reproduce: a NaN in the tensor operand comes out as NaN
                # (ugt x, c and ogt c, x), or is multiplied by x afterwards (the olt clamps of hard-swish / hard-sigmoid)
                first_is_tensor = isinstance(a_, tuple)
                if not ((c[1] == "ugt" and first_is_tensor) or (c[1] == "ogt" and not first_is_tensor) or c[1] == "olt"):
                    err(st, f"clamp written as cmpf {c[1]}: only cmpf ugt x, c / cmpf ogt c, x / cmpf olt are recognised")
                env[res] = ("max" if c[1] in ("ugt", "ogt") else "min", a_, b_)
            elif op == "arith.truncf":
                env[res] = get(operands[0])
            else:
                err(st, f"unsupported op {op} in an elementwise body")
        return commute(out)

    def apply_activation(st: Stmt, base: str, code: int, occurrences: int):
        v = val.get(base)
        if uses.get(base, 0) != occurrences:
            err(st, f"{base} feeds an activation but has other readers")
        if v and v[0] == "conv" and v[2] in ("bn", "add", "bias") and v[1].act == 0 and code in (1, 3):
            v[1].act = code
            v[1].relu = int(code == 1)
            val[st.result] = ("node", v[1])
        elif v and v[0] == "node" and v[1].kind == "fc" and v[1].act == 0 and v[1].b >= 0 and code in (1, 3):
            v[1].act = code
            val[st.result] = ("node", v[1])
        elif v and v[0] == "se1" and code == 1:
            val[st.result] = ("se1r",) + v[1:]
        elif v and v[0] == "se2" and code == 2:
            val[st.result] = ("gate",) + v[1:]
        else:
            err(st, "this activation does not follow a convolution, FC layer or squeeze-and-excitation stage it can fuse into")

    def elementwise(st: Stmt, ins, ops, arg):
        e = body_expr(st, ops, arg)
        names = sorted(set(leaves(e, [])))
        if len(names) == 1:
            ex = subst(e, names[0])
            n_occ = leaves(e, []).count(names[0])
            for code, pat in ((1, RELU), (3, HSWISH), (2, HSIGMOID)):
                if ex == pat:
                    # readers of the base tensor: one per generic of the chain that names it
                    return apply_activation(st, names[0], code, n_occ)
            if ex in PREFIXES:
                val[st.result] = ("ew", e)
                return
            v = val.get(names[0])
            if ex[0] == "div" and ex[1] == X and v and v[0] == "sumpool" and ex[2] == float(v[2]):
                single_use(st, names[0])
                val[st.result] = ("node", new_node("avgpool", inp=v[1]))
                return
            err(st, f"unrecognised elementwise function {ex}")
        if len(names) == 2 and e[0] == "add" and e[1][0] == "t" and e[2][0] == "t":
            a_, b_ = e[1][1], e[2][1]
            if len(shapes.get(a_, ())) == 4 and len(shapes.get(b_, ())) == 4:
                return residual_add(st, a_, b_)
            fcn, cn = (a_, b_) if b_ in consts else (b_, a_)
            v = val.get(fcn)
            if not v or v[0] != "fc" or cn not in consts or consts[cn][0] != (v[1].cout,):
                err(st, "a vector add is only recognised as the bias of the FC layer")
            single_use(st, fcn)
            v[1].b = consts[cn][1]
            val[st.result] = ("node", v[1])
            return
        if len(names) == 2 and e[0] == "mul" and e[1][0] == "t" and e[2][0] == "t":
            g, t = (e[1][1], e[2][1]) if val.get(e[1][1], ("",))[0] == "gate" else (e[2][1], e[1][1])
            gv = val.get(g)
            if not gv or gv[0] != "gate":
                err(st, "a product of two tensors is only recognised as squeeze-and-excitation scaling")
            single_use(st, g)
            pool = gv[1]
            src = tensor_of(st, t)
            if src == 0 or pool.inp is not src:
                err(st, "the squeeze-and-excitation gate must scale the tensor it was pooled from")
            nodes.remove(pool)
            n = new_node("se", inp=src, cin=gv[5], cout=gv[5], cr=gv[4], w=gv[2], b=gv[3], w2=gv[6], b2=gv[7])
            val[st.result] = ("node", n)
            return
        err(st, f"unrecognised linalg.generic body {[o[1] for o in ops]}")

    def residual_add(st: Stmt, x0: str, x1: str):
        # the operand that is an unfinished conv takes the other one in its epilogue
        a, b = val.get(x0), val.get(x1)

        def open_conv(v):
            return v and v[0] == "conv" and v[1].kind == "conv" and v[2] == "bn" and v[1].act == 0 and v[1].res is None

        main, other = (x0, x1) if open_conv(a) and uses.get(x0, 0) == 1 else (x1, x0)
        mv = val.get(main)
        if not open_conv(mv):
            err(st, "a residual add needs one operand that is a convolution + batch-norm without activation")
        single_use(st, main)
        ov = val.get(other)
        if ov and ov[0] == "conv" and uses.get(other, 0) == 1:      # the other branch ends here (downsample conv + batch-norm)
            val[other] = ("node", ov[1])
        mv[1].res = tensor_of(st, other)
        if mv[1].res == 0:
            err(st, "the network input cannot be a residual")
        val[st.result] = ("conv", mv[1], "add")

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
        elif st.op == "linalg.fill":
            ins, types = _operands(st.head, "ins")
            if ins and ins[0] in scalars and re.search(r"->\s*tensor<(i64|i32|f32)>", st.head):
                scalar_tensors[st.result] = scalars[ins[0]]     # rank-0 tensor holding a constant (the 6 of hard-swish)
            continue
        elif st.op in ("tensor.empty", "arith.cmpi", "cf.assert"):
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
            k, c, r, s_ = consts[ins[1]][0]
            if r != s_:
                err(st, "only square filters are supported")
            outs, _ = _operands(st.head, "outs")
            bias = val.get(outs[0]) if outs else None
            bias_off = consts[bias[1]][1] if bias and bias[0] == "bias_bcast" and consts[bias[1]][0] == (k,) else -1
            sv = val.get(src)
            if sv and sv[0] in ("node", "se1r") and r == 1 and bias_off >= 0 and \
                    (sv[0] == "se1r" or (sv[1].kind == "avgpool" and shapes.get(src, (0, 0, 0, 0))[2:] == (1, 1))):
                # the two 1x1 convolutions of a squeeze-and-excitation block run on the pooled [N,C,1,1] vector
                if sv[0] == "node":
                    single_use(st, src)
                    val[st.result] = ("se1", sv[1], consts[ins[1]][1], bias_off, k, c)
                else:
                    single_use(st, src)
                    if c != sv[4] or k != sv[5]:
                        err(st, "the second squeeze-and-excitation convolution must map the squeezed width back")
                    val[st.result] = ("se2", sv[1], sv[2], sv[3], sv[4], sv[5], consts[ins[1]][1], bias_off)
                shapes[st.result] = _shape(st.head.split("->")[-1])
                continue
            n = new_node("conv", inp=tensor_of(st, src), cin=c, cout=k, k=r, stride=stride, pad=pad, w=consts[ins[1]][1])
            if bias_off >= 0:
                n.b = bias_off
                val[st.result] = ("conv", n, "bias")
            else:
                val[st.result] = ("conv", n, "raw")
            shapes[st.result] = _shape(st.head.split("->")[-1])
        elif st.op == "linalg.depthwise_conv_2d_nchw_chw":
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
            wv = val.get(ins[1])
            if not wv or wv[0] != "const":
                err(st, "the depthwise filter must be a (collapsed) constant")
            wshape, woff = consts[wv[1]]
            ch, r, s_ = wshape[0], wshape[-2], wshape[-1]
            if r != s_ or math.prod(wshape) != ch * r * s_:
                err(st, "only square depthwise filters with one filter per channel are supported")
            n = new_node("dwconv", inp=tensor_of(st, src), cin=ch, cout=ch, k=r, stride=stride, pad=pad, w=woff)
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
                if eps is None or not (0.0 < eps < 1.0):
                    err(st, f"batch-norm eps {eps} is not a small positive constant")
                v = val.get(arg[x_arg])
                if not v or v[0] != "conv" or v[2] != "raw":
                    err(st, "batch-norm must follow a convolution directly")
                single_use(st, arg[x_arg])
                n = v[1]
                for role, a in (("gamma", gamma_arg), ("beta", beta_arg), ("mean", mean_arg), ("var", var_arg)):
                    if arg[a] not in consts or consts[arg[a]][0] != (n.cout,):
                        err(st, f"batch-norm {role} must be a constant of {n.cout} values")
                    setattr(n, role, consts[arg[a]][1])
                n.eps = float(eps)
                val[st.result] = ("conv", n, "bn")
            elif kinds == ["arith.sitofp", "linalg.yield"] and ins and ins[0] in scalar_tensors:
                scalar_tensors[st.result] = scalar_tensors[ins[0]]
            elif kinds == ["linalg.yield"] and len(ins) == 1 and ins[0] in consts and len(consts[ins[0]][0]) == 2:
                val[st.result] = ("const_t", ins[0])     # FC weight transposed at run time (Res18.mlir:617-620)
            elif kinds == ["linalg.yield"] and len(ins) == 1 and ins[0] in consts and len(consts[ins[0]][0]) == 1:
                val[st.result] = ("bias_bcast", ins[0])  # a bias vector broadcast into a convolution's init tensor
            else:
                elementwise(st, ins, ops, arg)
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
            if x == 0 or x.kind not in ("avgpool", "fc"):
                err(st, "an FC layer must read the global average pool or another FC layer")
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
        if (n.kind == "conv" and n.gamma < 0 and n.b < 0) or (n.kind == "dwconv" and n.gamma < 0):
            raise PlanImportError(f"convolution #{n.order} has neither batch-norm nor bias; plain convolutions are not in the recognised set")
        if n.kind == "fc" and n.b < 0:
            raise PlanImportError(f"FC layer #{n.order} has no bias")
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
