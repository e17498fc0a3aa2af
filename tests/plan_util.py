"""Helpers shared by the plan tests: a tiny generator of torch-mlir-style linalg text, a reader of
plan text, random parameters for a plan and a CPU interpreter of plans built from the oracle's ops
(test infrastructure only)."""
import math
import zlib

import numpy as np


def parse_plan_text(text):
    """Plan text -> (total, out_features, [dict per node])."""
    total = out = 0
    nodes = []
    for line in text.splitlines():
        t = line.split("#")[0].split()
        if not t or t[0] == "nncv_b200_plan":
            continue
        if t[0] == "params":
            total, out = int(t[1]), int(t[3])
            continue
        d = {"kind": t[0]}
        for f in t[1:]:
            k, v = f.split("=")
            d[k] = int(v)
        nodes.append(d)
    return total, out, nodes


def plan_tensors(nodes):
    """(offset, shape, role) of every parameter tensor a plan names, sorted by offset, duplicates merged."""
    seen = {}
    for n in nodes:
        if n["kind"] == "conv":
            seen.setdefault(n["w"], ((n["cout"], n["cin"], n["k"], n["k"]), "conv"))
            if "gamma" in n:
                for role in ("gamma", "beta", "mean", "var"):
                    seen.setdefault(n[role], ((n["cout"],), role))
        elif n["kind"] == "fc":
            seen.setdefault(n["w"], ((n["cout"], n["cin"]), "fcw"))
            seen.setdefault(n["b"], ((n["cout"],), "fcb"))
    return [(off, shape, role) for off, (shape, role) in sorted(seen.items())]


def random_blob(total, nodes, seed=0):
    """fp32 blob with the distributions the benchmark configs name, per tensor role."""
    blob = np.zeros(total, np.float32)
    pos = 0
    for off, shape, role in plan_tensors(nodes):
        assert off == pos, "the plan's tensors must tile the blob"
        g = np.random.Generator(np.random.Philox(key=[seed, zlib.crc32(f"{off}.{role}".encode())]))
        n = int(np.prod(shape))
        if role == "conv":
            v = g.standard_normal(n, dtype=np.float32) * np.float32(math.sqrt(2.0 / (shape[1] * shape[2] * shape[3])))
        elif role in ("gamma", "var"):
            v = g.uniform(0.5, 1.5, n).astype(np.float32)
        elif role in ("beta", "mean"):
            v = g.standard_normal(n, dtype=np.float32) * np.float32(0.1)
        else:
            b = 1.0 / math.sqrt(shape[-1] if role == "fcw" else n)
            v = g.uniform(-b, b, n).astype(np.float32)
        blob[off:off + n] = v
        pos += n
    assert pos == total
    return blob


def blob_indexers(nodes):
    """(name, shape) per tensor in blob order, for writing a model.bin that matches the plan."""
    return [(f"__constant_{'x'.join(map(str, shape))}xf32_{i}", shape) for i, (off, shape, role) in enumerate(plan_tensors(nodes))]


def run_plan_cpu(nodes, blob, x, ob, acc64=False):
    """Interprets a plan with the oracle's ops (conv -> batch-norm -> add -> ReLU, pools, FC)."""
    t = {0: np.ascontiguousarray(x, np.float32)}
    for n in nodes:
        a = t[n["in"]]
        if n["kind"] == "conv":
            co = n["cout"]
            w = blob[n["w"]:n["w"] + co * n["cin"] * n["k"] ** 2].reshape(co, n["cin"], n["k"], n["k"])
            y = ob.conv2d(a, w, n["stride"], n["pad"], acc64=acc64)
            if "gamma" in n:
                v = lambda r: blob[n[r]:n[r] + co]
                y = ob.batchnorm(y, v("gamma"), v("beta"), v("mean"), v("var"))
            if n.get("res", -1) >= 0:
                y = y + t[n["res"]]
            if n.get("relu"):
                y = ob.relu(y)
        elif n["kind"] == "maxpool":
            y = ob.maxpool(a, n["k"], n["stride"], n["pad"])
        elif n["kind"] == "avgpool":
            y = ob.avgpool_global(a)
        else:
            w = blob[n["w"]:n["w"] + n["cout"] * n["cin"]].reshape(n["cout"], n["cin"])
            y = ob.matmul(a, np.ascontiguousarray(w.T), blob[n["b"]:n["b"] + n["cout"]], False, acc64=acc64)
        t[n["id"]] = y
    return t[nodes[-1]["id"]]


# ---------------------------------------------------------------- synthetic linalg modules
class MlirBuilder:
    """Writes `@forward` in the style torch-mlir emits (the op spellings of nncv's tests/Nets/*.mlir)."""

    def __init__(self, n, h, w, ety="f32"):
        self.e = ety
        self.consts, self.body = [], []
        self.n, self.k = n, 0
        self.in_shape = (n, 3, h, w)

    def _v(self):
        self.k += 1
        return f"%v{self.k}"

    def const(self, shape):
        name = f"%cst_{len(self.consts)}"
        self.consts.append(f"    {name} = arith.constant dense_resource<__elided__> : {self.ty(shape)}")
        return name

    def ty(self, shape):
        return "tensor<" + "x".join(map(str, shape)) + f"x{self.e}>"

    def pad(self, src, shape, p, fill):
        out = shape[:2] + (shape[2] + 2 * p, shape[3] + 2 * p)
        r = self._v()
        self.body += [f"    {r} = tensor.pad {src} low[0, 0, {p}, {p}] high[0, 0, {p}, {p}] {{",
                      "    ^bb0(%arg1: index, %arg2: index, %arg3: index, %arg4: index):",
                      f"      tensor.yield {fill} : {self.e}", f"    }} : {self.ty(shape)} to {self.ty(out)}"]
        return r, out

    def conv_bn(self, src, shape, cout, k, stride, p, bn_order=("gamma", "beta", "mean", "var")):
        if p:
            src, shape = self.pad(src, shape, p, "%zero")
        w = self.const((cout, shape[1], k, k))
        oh, ow = (shape[2] - k) // stride + 1, (shape[3] - k) // stride + 1
        out = (shape[0], cout, oh, ow)
        e, f, c = self._v(), self._v(), self._v()
        self.body += [f"    {e} = tensor.empty() : {self.ty(out)}",
                      f"    {f} = linalg.fill ins(%zero : {self.e}) outs({e} : {self.ty(out)}) -> {self.ty(out)}",
                      f"    {c} = linalg.conv_2d_nchw_fchw {{dilations = dense<1> : vector<2xi64>, strides = dense<{stride}> : vector<2xi64>}} "
                      f"ins({src}, {w} : {self.ty(shape)}, {self.ty((cout, shape[1], k, k))}) outs({f} : {self.ty(out)}) -> {self.ty(out)}"]
        vec = {r: self.const((cout,)) for r in ("beta", "gamma", "var", "mean")}   # declaration order != operand order
        names = {r: f"%in_{i}" for i, r in enumerate(bn_order)}
        b = self._v()
        ins = ", ".join([c] + [vec[r] for r in bn_order])
        types = ", ".join([self.ty(out)] + [self.ty((cout,))] * 4)
        args = ", ".join([f"%in: {self.e}"] + [f"{names[r]}: {self.e}" for r in bn_order] + [f"%out: {self.e}"])
        self.body += [f"    {b} = linalg.generic {{indexing_maps = [#map, #map1, #map1, #map1, #map1, #map], iterator_types = [\"parallel\", \"parallel\", \"parallel\", \"parallel\"]}} "
                      f"ins({ins} : {types}) outs({c} : {self.ty(out)}) {{",
                      f"    ^bb0({args}):",
                      f"      %90 = arith.truncf %eps : f64 to {self.e}", f"      %91 = arith.addf {names['var']}, %90 : {self.e}",
                      f"      %92 = math.rsqrt %91 : {self.e}", f"      %93 = arith.subf %in, {names['mean']} : {self.e}",
                      f"      %94 = arith.mulf %93, %92 : {self.e}", f"      %95 = arith.mulf %94, {names['gamma']} : {self.e}",
                      f"      %96 = arith.addf %95, {names['beta']} : {self.e}", f"      linalg.yield %96 : {self.e}",
                      f"    }} -> {self.ty(out)}"]
        return b, out

    def relu(self, src, shape):
        r = self._v()
        self.body += [f"    {r} = linalg.generic {{indexing_maps = [#map2, #map], iterator_types = [\"parallel\", \"parallel\", \"parallel\", \"parallel\"]}} "
                      f"ins({src} : {self.ty(shape)}) outs({src} : {self.ty(shape)}) {{",
                      f"    ^bb0(%in: {self.e}, %out: {self.e}):", f"      %90 = arith.cmpf ugt, %in, %zero : {self.e}",
                      f"      %91 = arith.select %90, %in, %zero : {self.e}", f"      linalg.yield %91 : {self.e}", f"    }} -> {self.ty(shape)}"]
        return r

    def add(self, a, b, shape):
        r = self._v()
        self.body += [f"    {r} = linalg.generic {{indexing_maps = [#map2, #map2, #map], iterator_types = [\"parallel\", \"parallel\", \"parallel\", \"parallel\"]}} "
                      f"ins({a}, {b} : {self.ty(shape)}, {self.ty(shape)}) outs({a} : {self.ty(shape)}) {{",
                      f"    ^bb0(%in: {self.e}, %in_9: {self.e}, %out: {self.e}):", f"      %90 = arith.addf %in, %in_9 : {self.e}",
                      f"      linalg.yield %90 : {self.e}", f"    }} -> {self.ty(shape)}"]
        return r

    def maxpool(self, src, shape, k, stride, p):
        if p:
            src, shape = self.pad(src, shape, p, "%ninf")
        out = shape[:2] + ((shape[2] - k) // stride + 1, (shape[3] - k) // stride + 1)
        e, f, wn, r = self._v(), self._v(), self._v(), self._v()
        self.body += [f"    {e} = tensor.empty() : {self.ty(out)}",
                      f"    {f} = linalg.fill ins(%ninf : {self.e}) outs({e} : {self.ty(out)}) -> {self.ty(out)}",
                      f"    {wn} = tensor.empty() : {self.ty((k, k))}",
                      f"    {r} = linalg.pooling_nchw_max {{dilations = dense<1> : vector<2xi64>, strides = dense<{stride}> : vector<2xi64>}} "
                      f"ins({src}, {wn} : {self.ty(shape)}, {self.ty((k, k))}) outs({f} : {self.ty(out)}) -> {self.ty(out)}"]
        return r, out

    def head(self, src, shape, classes):
        n, c, h, w = shape
        o1 = (n, c, 1, 1)
        e, f, wn, s, d, col, wt_e, wt, oe, of, mm, r = (self._v() for _ in range(12))
        fcw, fcb = self.const((classes, c)), self.const((classes,))
        self.extra = f"    %hw = arith.constant {float(h * w):e} : {self.e}"
        self.body += [f"    {e} = tensor.empty() : {self.ty(o1)}",
                      f"    {f} = linalg.fill ins(%zero : {self.e}) outs({e} : {self.ty(o1)}) -> {self.ty(o1)}",
                      f"    {wn} = tensor.empty() : {self.ty((h, w))}",
                      f"    {s} = linalg.pooling_nchw_sum {{dilations = dense<1> : vector<2xi64>, strides = dense<1> : vector<2xi64>}} "
                      f"ins({src}, {wn} : {self.ty(shape)}, {self.ty((h, w))}) outs({f} : {self.ty(o1)}) -> {self.ty(o1)}",
                      f"    {d} = linalg.generic {{indexing_maps = [#map, #map], iterator_types = [\"parallel\", \"parallel\", \"parallel\", \"parallel\"]}} "
                      f"ins({s} : {self.ty(o1)}) outs({e} : {self.ty(o1)}) {{", f"    ^bb0(%in: {self.e}, %out: {self.e}):",
                      f"      %90 = arith.divf %in, %hw : {self.e}", f"      linalg.yield %90 : {self.e}", f"    }} -> {self.ty(o1)}",
                      f"    {col} = tensor.collapse_shape {d} [[0], [1, 2, 3]] : {self.ty(o1)} into {self.ty((n, c))}",
                      f"    {wt_e} = tensor.empty() : {self.ty((c, classes))}",
                      f"    {wt} = linalg.generic {{indexing_maps = [#map3, #map4], iterator_types = [\"parallel\", \"parallel\"]}} "
                      f"ins({fcw} : {self.ty((classes, c))}) outs({wt_e} : {self.ty((c, classes))}) {{",
                      f"    ^bb0(%in: {self.e}, %out: {self.e}):", f"      linalg.yield %in : {self.e}", f"    }} -> {self.ty((c, classes))}",
                      f"    {oe} = tensor.empty() : {self.ty((n, classes))}",
                      f"    {of} = linalg.fill ins(%zero : {self.e}) outs({oe} : {self.ty((n, classes))}) -> {self.ty((n, classes))}",
                      f"    {mm} = linalg.matmul ins({col}, {wt} : {self.ty((n, c))}, {self.ty((c, classes))}) outs({of} : {self.ty((n, classes))}) -> {self.ty((n, classes))}",
                      f"    {r} = linalg.generic {{indexing_maps = [#map5, #map6, #map3], iterator_types = [\"parallel\", \"parallel\"]}} "
                      f"ins({mm}, {fcb} : {self.ty((n, classes))}, {self.ty((classes,))}) outs({oe} : {self.ty((n, classes))}) {{",
                      f"    ^bb0(%in: {self.e}, %in_9: {self.e}, %out: {self.e}):", f"      %90 = arith.addf %in, %in_9 : {self.e}",
                      f"      linalg.yield %90 : {self.e}", f"    }} -> {self.ty((n, classes))}",
                      f"    return {r} : {self.ty((n, classes))}"]
        self.out_ty = self.ty((n, classes))

    def text(self):
        head = ["module {", f"  func.func @forward(%arg0: {self.ty(self.in_shape)}) -> {self.out_ty} {{"]
        scal = [f"    %zero = arith.constant 0.000000e+00 : {self.e}",
                f"    %ninf = arith.constant {'0xFF800000' if self.e == 'f32' else '0xFC00'} : {self.e}",
                "    %eps = arith.constant 1.000000e-05 : f64", getattr(self, "extra", "")]
        return "\n".join(head + self.consts + scal + self.body + ["  }", "}"]) + "\n"


def small_net_mlir(n=2, h=40, w=56, classes=10, bn_order=("gamma", "beta", "mean", "var")):
    """A small non-ResNet module: conv3x3 s1 (3->16) -> max-pool 2x2 s2 -> residual pair of 3x3 convs (64 ch after a
    strided 3x3) with a 1x1 stride-2 projection -> conv 1x1 -> global average pool -> FC."""
    b = MlirBuilder(n, h, w)
    x, s = b.conv_bn("%arg0", b.in_shape, 16, 3, 1, 1, bn_order)
    x = b.relu(x, s)
    x, s = b.maxpool(x, s, 2, 2, 0)
    t, st = b.conv_bn(x, s, 64, 3, 2, 1, bn_order)
    t = b.relu(t, st)
    u, su = b.conv_bn(t, st, 64, 3, 1, 1, bn_order)
    d, sd = b.conv_bn(x, s, 64, 1, 2, 0, bn_order)
    y = b.relu(b.add(u, d, su), su)
    z, sz = b.conv_bn(y, su, 128, 1, 1, 0, bn_order)
    z = b.relu(z, sz)
    v, sv = b.conv_bn(z, sz, 128, 3, 1, 1, bn_order)
    y2 = b.relu(b.add(v, z, sv), sv)
    b.head(y2, sv, classes)
    return b.text()
