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
            elif "b" in n:
                seen.setdefault(n["b"], ((n["cout"],), "fcb"))
        elif n["kind"] == "dwconv":
            seen.setdefault(n["w"], ((n["c"], 1, n["k"], n["k"]), "conv"))
            for role in ("gamma", "beta", "mean", "var"):
                seen.setdefault(n[role], ((n["c"],), role))
        elif n["kind"] == "se":
            seen.setdefault(n["w1"], ((n["cr"], n["c"], 1, 1), "conv"))
            seen.setdefault(n["b1"], ((n["cr"],), "fcb"))
            seen.setdefault(n["w2"], ((n["c"], n["cr"], 1, 1), "conv"))
            seen.setdefault(n["b2"], ((n["c"],), "fcb"))
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


ACT_NAMES = {0: "none", 1: "relu", 2: "hard_sigmoid", 3: "hard_swish", 4: "sigmoid", 5: "silu"}


def _eps(n):
    if "eps_bits" not in n:
        return 1e-5
    return float(np.array([n["eps_bits"]], np.uint32).view(np.float32)[0])


def _bn(y, n, blob, c):
    v = lambda r: blob[n[r]:n[r] + c].astype(np.float32)
    rs = (1.0 / np.sqrt(v("var") + np.float32(_eps(n)))).astype(np.float32)
    return ((y - v("mean")[None, :, None, None]) * rs[None, :, None, None] * v("gamma")[None, :, None, None]
            + v("beta")[None, :, None, None]).astype(np.float32)


def run_plan_cpu(nodes, blob, x, ob, acc64=False):
    """Interprets a plan with the oracle's ops (conv / depthwise conv -> batch-norm -> add -> activation,
    squeeze-and-excitation, pools, FC layers)."""
    t = {0: np.ascontiguousarray(x, np.float32)}
    for n in nodes:
        a = t[n["in"]]
        act = n.get("act", 1 if n.get("relu") else 0)
        if n["kind"] == "conv":
            co = n["cout"]
            w = blob[n["w"]:n["w"] + co * n["cin"] * n["k"] ** 2].reshape(co, n["cin"], n["k"], n["k"])
            y = ob.conv2d(a, w, n["stride"], n["pad"], acc64=acc64)
            if "gamma" in n:
                y = _bn(y, n, blob, co) if "eps_bits" in n else ob.batchnorm(y, *(blob[n[r]:n[r] + co] for r in ("gamma", "beta", "mean", "var")))
            elif "b" in n:
                y = y + blob[n["b"]:n["b"] + co][None, :, None, None]
            if n.get("res", -1) >= 0:
                y = y + t[n["res"]]
            if act:
                y = ob.relu(y) if act == 1 else ob.activation(y, ACT_NAMES[act])
        elif n["kind"] == "dwconv":
            c, k = n["c"], n["k"]
            w = blob[n["w"]:n["w"] + c * k * k].reshape(c, k, k)
            y = _bn(ob.depthwise_conv2d(a, w, n["stride"], n["pad"], acc64=acc64), n, blob, c)
            if act:
                y = ob.activation(y, ACT_NAMES[act])
        elif n["kind"] == "se":
            c, cr = n["c"], n["cr"]
            w1 = blob[n["w1"]:n["w1"] + cr * c].reshape(cr, c)
            w2 = blob[n["w2"]:n["w2"] + cr * c].reshape(c, cr)
            gate = ob.se_gate(ob.avgpool_global(a), w1, blob[n["b1"]:n["b1"] + cr], w2, blob[n["b2"]:n["b2"] + c])
            y = (a * gate[:, :, None, None]).astype(np.float32)
        elif n["kind"] == "maxpool":
            y = ob.maxpool(a, n["k"], n["stride"], n["pad"])
        elif n["kind"] == "avgpool":
            y = ob.avgpool_global(a)
        else:
            w = blob[n["w"]:n["w"] + n["cout"] * n["cin"]].reshape(n["cout"], n["cin"])
            y = ob.matmul(a, np.ascontiguousarray(w.T), blob[n["b"]:n["b"] + n["cout"]], False, acc64=acc64)
            if act:
                y = ob.activation(y, ACT_NAMES[act])
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
        self.scalars_extra = []
        self.eps = 1e-5

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

    # ---- the op spellings of tests/Nets/MobileNetV3.mlir -----------------------------------------
    PAR4 = 'iterator_types = ["parallel", "parallel", "parallel", "parallel"]'
    PAR2 = 'iterator_types = ["parallel", "parallel"]'

    def _ew(self, ins, types, body, out_ty, maps, par=None):
        """One linalg.generic with the given region lines; block arguments are %in, %in_1, ..."""
        r = self._v()
        args = ", ".join([f"%in{'' if i == 0 else '_' + str(i)}: {self.e}" for i in range(len(ins))] + [f"%out: {self.e}"])
        self.body += [f"    {r} = linalg.generic {{indexing_maps = [{maps}], {par or self.PAR4}}} ins({', '.join(ins)} : {', '.join(types)}) "
                      f"outs(%dst : {out_ty}) {{", f"    ^bb0({args}):"] + [f"      {b}" for b in body] + [f"    }} -> {out_ty}"]
        return r

    def scalar_tensor(self, value):
        """A rank-0 f32 tensor holding an integer constant: fill of tensor<i64> + sitofp generic (MobileNetV3.mlir:267-276)."""
        c, f, r = self._v(), self._v(), self._v()
        self.body += [f"    {c} = arith.constant {int(value)} : i64",
                      f"    {f} = linalg.fill ins({c} : i64) outs(%e : tensor<i64>) -> tensor<i64>",
                      f"    {r} = linalg.generic {{indexing_maps = [#map3, #map3], iterator_types = []}} ins({f} : tensor<i64>) outs(%e2 : tensor<{self.e}>) {{",
                      f"    ^bb0(%in: i64, %out: {self.e}):", f"      %90 = arith.sitofp %in : i64 to {self.e}", f"      linalg.yield %90 : {self.e}",
                      f"    }} -> tensor<{self.e}>"]
        return r

    def hardswish(self, x, shape):
        """x * min(max(x + 3, 0), 6) / 6 over five generics (MobileNetV3.mlir:263-295); works on 4-D and 2-D values."""
        ty, e = self.ty(shape), self.e
        par = self.PAR4 if len(shape) == 4 else self.PAR2
        six = self.scalar_tensor(6)
        a = self._ew([x], [ty], [f"%90 = arith.addf %in, %three : {e}", f"linalg.yield %90 : {e}"], ty, "#map2, #map", par)
        b = self._ew([a], [ty], [f"%90 = arith.cmpf ugt, %in, %zero : {e}", f"%91 = arith.select %90, %in, %zero : {e}", f"linalg.yield %91 : {e}"],
                     ty, "#map2, #map", par)
        c = self._ew([b, six], [ty, f"tensor<{e}>"], [f"%90 = arith.cmpf olt, %in, %in_1 : {e}", f"%91 = arith.select %90, %in, %in_1 : {e}",
                                                      f"linalg.yield %91 : {e}"], ty, "#map2, #map4, #map", par)
        d = self._ew([c], [ty], [f"%90 = arith.divf %in, %sixf : {e}", f"linalg.yield %90 : {e}"], ty, "#map2, #map", par)
        return self._ew([d, x], [ty, ty], [f"%90 = arith.mulf %in, %in_1 : {e}", f"linalg.yield %90 : {e}"], ty, "#map2, #map2, #map", par)

    def hardsigmoid(self, x, shape):
        """max(min((x + 3) / 6, 1), 0) with the constants as rank-0 tensors in first position (MobileNetV3.mlir:345-383)."""
        ty, e = self.ty(shape), self.e
        one, zero = self.scalar_tensor(1), self.scalar_tensor(0)
        a = self._ew([x], [ty], [f"%90 = arith.addf %in, %three : {e}", f"linalg.yield %90 : {e}"], ty, "#map5, #map")
        b = self._ew([a], [ty], [f"%90 = arith.divf %in, %sixf : {e}", f"linalg.yield %90 : {e}"], ty, "#map5, #map")
        c = self._ew([one, b], [f"tensor<{e}>", ty], [f"%90 = arith.cmpf olt, %in, %in_1 : {e}", f"%91 = arith.select %90, %in, %in_1 : {e}",
                                                      f"linalg.yield %91 : {e}"], ty, "#map4, #map5, #map")
        return self._ew([zero, c], [f"tensor<{e}>", ty], [f"%90 = arith.cmpf ogt, %in, %in_1 : {e}", f"%91 = arith.select %90, %in, %in_1 : {e}",
                                                          f"linalg.yield %91 : {e}"], ty, "#map4, #map5, #map")

    def _bn(self, c, out, ch, bn_order):
        vec = {r: self.const((ch,)) for r in ("beta", "gamma", "var", "mean")}
        names = {r: f"%in_{i}" for i, r in enumerate(bn_order)}
        b = self._v()
        ins = ", ".join([c] + [vec[r] for r in bn_order])
        types = ", ".join([self.ty(out)] + [self.ty((ch,))] * 4)
        args = ", ".join([f"%in: {self.e}"] + [f"{names[r]}: {self.e}" for r in bn_order] + [f"%out: {self.e}"])
        self.body += [f"    {b} = linalg.generic {{indexing_maps = [#map, #map1, #map1, #map1, #map1, #map], {self.PAR4}}} "
                      f"ins({ins} : {types}) outs({c} : {self.ty(out)}) {{", f"    ^bb0({args}):",
                      f"      %90 = arith.truncf %eps : f64 to {self.e}", f"      %91 = arith.addf {names['var']}, %90 : {self.e}",
                      f"      %92 = math.rsqrt %91 : {self.e}", f"      %93 = arith.subf %in, {names['mean']} : {self.e}",
                      f"      %94 = arith.mulf %93, %92 : {self.e}", f"      %95 = arith.mulf %94, {names['gamma']} : {self.e}",
                      f"      %96 = arith.addf %95, {names['beta']} : {self.e}", f"      linalg.yield %96 : {self.e}", f"    }} -> {self.ty(out)}"]
        return b

    def dwconv_bn(self, src, shape, k, stride, p, bn_order=("gamma", "beta", "mean", "var")):
        if p:
            src, shape = self.pad(src, shape, p, "%zero")
        ch = shape[1]
        w = self.const((ch, 1, k, k))
        out = (shape[0], ch, (shape[2] - k) // stride + 1, (shape[3] - k) // stride + 1)
        col, c = self._v(), self._v()
        self.body += [f"    {col} = tensor.collapse_shape {w} [[0, 1], [2], [3]] : {self.ty((ch, 1, k, k))} into {self.ty((ch, k, k))}",
                      f"    {c} = linalg.depthwise_conv_2d_nchw_chw {{dilations = dense<1> : vector<2xi64>, strides = dense<{stride}> : vector<2xi64>}} "
                      f"ins({src}, {col} : {self.ty(shape)}, {self.ty((ch, k, k))}) outs(%dst : {self.ty(out)}) -> {self.ty(out)}"]
        return self._bn(c, out, ch, bn_order), out

    def conv_bias(self, src, shape, cout):
        """1x1 convolution whose init tensor is the broadcast bias (MobileNetV3.mlir:325-331)."""
        w, bias = self.const((cout, shape[1], 1, 1)), self.const((cout,))
        out = (shape[0], cout, shape[2], shape[3])
        bc = self._ew([bias], [self.ty((cout,))], [f"linalg.yield %in : {self.e}"], self.ty(out), "#map1, #map")
        c = self._v()
        self.body += [f"    {c} = linalg.conv_2d_nchw_fchw {{dilations = dense<1> : vector<2xi64>, strides = dense<1> : vector<2xi64>}} "
                      f"ins({src}, {w} : {self.ty(shape)}, {self.ty((cout, shape[1], 1, 1))}) outs({bc} : {self.ty(out)}) -> {self.ty(out)}"]
        return c, out

    def pool_mean(self, src, shape):
        n, c, h, w = shape
        o1 = (n, c, 1, 1)
        wn, sm = self._v(), self._v()
        hw = f"%hw{len(self.scalars_extra)}"
        self.scalars_extra.append(f"    {hw} = arith.constant {float(h * w):e} : {self.e}")
        self.body += [f"    {wn} = tensor.empty() : {self.ty((h, w))}",
                      f"    {sm} = linalg.pooling_nchw_sum {{dilations = dense<1> : vector<2xi64>, strides = dense<1> : vector<2xi64>}} "
                      f"ins({src}, {wn} : {self.ty(shape)}, {self.ty((h, w))}) outs(%dst : {self.ty(o1)}) -> {self.ty(o1)}"]
        d = self._ew([sm], [self.ty(o1)], [f"%90 = arith.divf %in, {hw} : {self.e}", f"linalg.yield %90 : {self.e}"], self.ty(o1), "#map, #map")
        return d, o1

    def se(self, x, shape, cr):
        """Squeeze-and-excitation (MobileNetV3.mlir:319-389)."""
        p1, s1 = self.pool_mean(x, shape)
        h, sh = self.conv_bias(p1, s1, cr)
        h = self._ew([h], [self.ty(sh)], [f"%90 = arith.cmpf ugt, %in, %zero : {self.e}", f"%91 = arith.select %90, %in, %zero : {self.e}",
                                          f"linalg.yield %91 : {self.e}"], self.ty(sh), "#map5, #map")
        g, sg = self.conv_bias(h, sh, shape[1])
        g = self.hardsigmoid(g, sg)
        return self._ew([g, x], [self.ty(sg), self.ty(shape)], [f"%90 = arith.mulf %in, %in_1 : {self.e}", f"linalg.yield %90 : {self.e}"],
                        self.ty(shape), "#map5, #map2, #map")

    def fc(self, x, n, cin, cout):
        """transpose generic -> matmul -> bias add on a [n, cin] value."""
        w, bias = self.const((cout, cin)), self.const((cout,))
        wt = self._ew([w], [self.ty((cout, cin))], [f"linalg.yield %in : {self.e}"], self.ty((cin, cout)), "#map6, #map7", self.PAR2)
        mm = self._v()
        self.body += [f"    {mm} = linalg.matmul ins({x}, {wt} : {self.ty((n, cin))}, {self.ty((cin, cout))}) outs(%dst : {self.ty((n, cout))}) -> {self.ty((n, cout))}"]
        return self._ew([mm, bias], [self.ty((n, cout)), self.ty((cout,))], [f"%90 = arith.addf %in, %in_1 : {self.e}", f"linalg.yield %90 : {self.e}"],
                        self.ty((n, cout)), "#map8, #map9, #map6", self.PAR2)

    def mobile_head(self, src, shape, hidden, classes):
        """global average pool -> FC + hard-swish -> FC (MobileNetV3.mlir:1774-1865)."""
        n, c = shape[0], shape[1]
        p1, s1 = self.pool_mean(src, shape)
        col = self._v()
        self.body += [f"    {col} = tensor.collapse_shape {p1} [[0], [1, 2, 3]] : {self.ty(s1)} into {self.ty((n, c))}"]
        h = self.hardswish(self.fc(col, n, c, hidden), (n, hidden))
        r = self.fc(h, n, hidden, classes)
        self.body += [f"    return {r} : {self.ty((n, classes))}"]
        self.out_ty = self.ty((n, classes))

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
                f"    %three = arith.constant 3.000000e+00 : {self.e}", f"    %sixf = arith.constant 6.000000e+00 : {self.e}",
                f"    %eps = arith.constant {self.eps:e} : f64", getattr(self, "extra", "")] + self.scalars_extra
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


def small_mobile_mlir(n=2, h=64, w=48, classes=10, eps=1e-3):
    """A small MobileNetV3-style module in the fixture's spellings: conv 3x3 s2 + BN + hard-swish -> depthwise 3x3 s2 + BN + ReLU ->
    SE -> 1x1 project (no activation) -> 1x1 expand + ReLU -> depthwise 5x5 + BN + hard-swish -> SE -> 1x1 project + residual ->
    1x1 + BN + hard-swish -> global average pool -> FC + hard-swish -> FC."""
    b = MlirBuilder(n, h, w)
    b.eps = eps
    x, s = b.conv_bn("%arg0", b.in_shape, 16, 3, 2, 1)
    x = b.hardswish(x, s)
    d, sd = b.dwconv_bn(x, s, 3, 2, 1)
    d = b.relu(d, sd)
    d = b.se(d, sd, 8)
    p, sp = b.conv_bn(d, sd, 24, 1, 1, 0)
    e, se_ = b.conv_bn(p, sp, 72, 1, 1, 0)
    e = b.relu(e, se_)
    f, sf = b.dwconv_bn(e, se_, 5, 1, 2)
    f = b.hardswish(f, sf)
    f = b.se(f, sf, 24)
    q, sq = b.conv_bn(f, sf, 24, 1, 1, 0)
    y = b.add(q, p, sq)
    z, sz = b.conv_bn(y, sq, 96, 1, 1, 0)
    z = b.hardswish(z, sz)
    b.mobile_head(z, sz, 128, classes)
    return b.text()
