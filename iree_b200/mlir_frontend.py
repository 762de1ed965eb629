"""Contraction dispatches from linalg-on-tensors MLIR text.

The compiler plugin (``compiler_plugin/src/RewriteContractionsPass.cpp``) matches these groups on
the IR; this module applies the same rules to the *text* of a function and yields the host plan
(``dispatch_gen.Plan``) the plugin's output corresponds to, so that the five benchmark programs
can be lowered and run here, where no ``iree-compile`` exists. It is a matcher for the handful of
op shapes below, not an MLIR parser:

  A/B  ``linalg.fill(0)`` -> ``linalg.matmul`` / ``linalg.batch_matmul`` (f16 or bf16 operands, f32
       accumulator) [-> elementwise generic whose body is one ``arith.truncf``]
  C    the same with i8 operands and an i32 accumulator [-> elementwise generic
       ``sitofp, mulf a_scale[d0], mulf w_scale[d1], truncf``]: the consumer that dispatch formation
       fuses into the matmul's dispatch (Dialect/Flow/Transforms/FormDispatchRegions.cpp:534-620)
  D    a dequantisation generic ``extsi i4, sitofp -> f16, mulf scale[n, g]`` (cloned into its
       consumer's dispatch, RegionOpUtils.cpp:530-610) feeding a contraction generic with two
       reduction dimensions (g, k) ``extf, extf, mulf, addf`` and a truncf consumer: the IR shape
       pinned by Dialect/Flow/Transforms/test/pipeline_tests.mlir:53-99. The i4 tensor may arrive
       as bytes through ``flow.tensor.bitcast`` (the Torch frontend's bitcast_quant_tensor).

``config_mlir`` writes the benchmark configurations in exactly these shapes.
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Tuple

from . import dispatch_gen as dg

_TENSOR = re.compile(r"tensor<((?:\d+x)*)(\w+)>")


def _tensor(text: str) -> Tuple[List[int], str]:
    m = _TENSOR.search(text)
    if not m:
        raise ValueError("not a static ranked tensor type: %r" % text)
    dims = [int(d) for d in m.group(1).split("x") if d]
    return dims, m.group(2)


class _Op:
    def __init__(self, result, name, ins, in_types, outs, out_types, attrs, body, result_type):
        self.result, self.name, self.ins, self.in_types = result, name, ins, in_types
        self.outs, self.out_types, self.attrs, self.body, self.result_type = outs, out_types, attrs, body, result_type


def _split_top(text: str) -> List[str]:
    parts, depth, cur = [], 0, ""
    for ch in text:
        if ch in "<([{":
            depth += 1
        elif ch in ">)]}":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        parts.append(cur.strip())
    return parts


def _parse_ins_outs(text: str, key: str):
    """Operand names and types of an `ins(...)` / `outs(...)` clause: `ins(%a, %b : type, type)`."""
    at = text.find(key + "(")
    if at < 0:
        return [], []
    i = at + len(key) + 1
    depth, k = 1, i
    while depth and k < len(text):
        depth += {"(": 1, ")": -1}.get(text[k], 0)
        k += 1
    names, _, types = text[i:k - 1].partition(":")
    return [x.strip() for x in names.split(",") if x.strip()], _split_top(types)


def _functions(text: str):
    for m in re.finditer(r"util\.func\s+(?:public\s+)?@(\w+)\((.*?)\)\s*->\s*(\(?[^{]*?\)?)\s*\{", text, re.S):
        start = m.end()
        depth, i = 1, start
        while depth and i < len(text):
            depth += {"{": 1, "}": -1}.get(text[i], 0)
            i += 1
        args = []
        for a in _split_top(m.group(2)):
            name, _, ty = a.partition(":")
            args.append((name.strip(), ty.strip()))
        yield m.group(1), args, text[start:i - 1]


def _ops(body: str) -> List[_Op]:
    ops = []
    pos = 0
    stmt = re.compile(r"(%[\w.]+)\s*=\s*([\w.]+)")
    while True:
        m = stmt.search(body, pos)
        if not m:
            break
        name = m.group(2)
        start = m.end()
        if name == "linalg.generic":
            # attribute dict, ins/outs, then a region, then "-> type"
            brace = body.index("{", start)
            depth, i = 1, brace + 1
            while depth:
                depth += {"{": 1, "}": -1}.get(body[i], 0)
                i += 1
            attrs = body[brace:i]
            region_start = body.index("{", i)
            head = body[i:region_start]
            depth, k = 1, region_start + 1
            while depth:
                depth += {"{": 1, "}": -1}.get(body[k], 0)
                k += 1
            region = body[region_start:k]
            tail = re.match(r"\s*->\s*(tensor<[^>]*>)", body[k:])
            ins, in_types = _parse_ins_outs(head, "ins")
            outs, out_types = _parse_ins_outs(head, "outs")
            body_ops = re.findall(r"=\s*(arith\.\w+)", region)
            ops.append(_Op(m.group(1), name, ins, in_types, outs, out_types, attrs, body_ops, tail.group(1) if tail else ""))
            pos = k
            continue
        end = body.find("\n", start)
        # statements may continue on following lines until the next "%x =" or "util.return"
        nxt = stmt.search(body, start)
        ret = body.find("util.return", start)
        limit = min(x for x in (nxt.start() if nxt else len(body), ret if ret >= 0 else len(body)))
        line = body[start:limit]
        ins, in_types = _parse_ins_outs(line, "ins")
        outs, out_types = _parse_ins_outs(line, "outs")
        rt = re.findall(r"->\s*(tensor<[^>]*>)", line)
        ops.append(_Op(m.group(1), name, ins, in_types, outs, out_types, line, [], rt[-1] if rt else ""))
        pos = limit if limit > start else end
    return ops


def _iterators(attrs: str) -> List[str]:
    m = re.search(r"iterator_types\s*=\s*\[([^\]]*)\]", attrs)
    return re.findall(r'"(\w+)"', m.group(1)) if m else []


def _maps(attrs: str, text: str) -> List[str]:
    """Result expressions of the op's indexing maps, e.g. ['d0,d1', 'd0', 'd1', 'd0,d1']; maps may be
    written inline or as references to `#name = affine_map<...>` definitions of the module."""
    m = re.search(r"indexing_maps\s*=\s*\[(.*?)\]\s*,\s*iterator_types", attrs, re.S)
    if not m:
        return []
    out = []
    for item in re.findall(r"affine_map<\([^)]*\)\s*->\s*\([^)]*\)>|#\w+", m.group(1)):
        if item.startswith("#"):
            d = re.search(re.escape(item) + r"\s*=\s*affine_map<\([^)]*\)\s*->\s*\(([^)]*)\)>", text)
            out.append(d.group(1).replace(" ", "") if d else "?")
        else:
            out.append(re.search(r"->\s*\(([^)]*)\)", item).group(1).replace(" ", ""))
    return out


def plans_from_mlir(text: str, device_tensor_maps: bool = True, sm_count: int = dg.SM_COUNT) -> Dict[str, dg.Plan]:
    """One plan per ``util.func`` of the module text that holds a contraction group."""
    plans = {}
    for fname, args, body in _functions(text):
        ops = _ops(body)
        by_result = {o.result: o for o in ops}
        arg_names = [a for a, _ in args]

        def users(v):
            return [o for o in ops if v in o.ins]

        def zero_fill(v):
            o = by_result.get(v)
            if not o or o.name != "linalg.fill":
                return False
            c = by_result.get(o.ins[0]) if o.ins else None
            return bool(c and c.name == "arith.constant" and re.search(r"constant\s+0(\.0*(e[+-]?0+)?)?\s*:", "constant" + c.attrs))

        def consumer(v, body_ops):
            u = users(v)
            if len(u) != 1 or u[0].name != "linalg.generic" or "reduction" in _iterators(u[0].attrs):
                return None
            return u[0] if u[0].body == body_ops else None

        plan = None
        for o in ops:
            if o.name in ("linalg.matmul", "linalg.batch_matmul"):
                (ld, lt), (rd, rt_), (ad, at) = _tensor(o.in_types[0]), _tensor(o.in_types[1]), _tensor(o.out_types[0])
                kind = {"f16": "f16", "bf16": "bf16", "i8": "i8"}.get(lt)
                if not kind or rt_ != lt or at != ("i32" if kind == "i8" else "f32") or not zero_fill(o.outs[0]):
                    continue
                batched = o.name == "linalg.batch_matmul"
                batch = ld[0] if batched else 1
                M, K, N = ld[-2], ld[-1], rd[-1]
                if o.ins != arg_names[:2]:
                    raise ValueError("@%s: matmul operands must be the function's first two arguments" % fname)
                epilogue = "acc"
                if kind != "i8":
                    t = consumer(o.result, ["arith.truncf"])
                    if t is not None and _tensor(t.result_type)[1] == kind:
                        epilogue = "cast"
                else:
                    q = consumer(o.result, ["arith.sitofp", "arith.mulf", "arith.mulf", "arith.truncf"])
                    if q is not None and len(q.ins) == 3 and _tensor(q.result_type)[1] == "f16":
                        maps = _maps(q.attrs, text)
                        sd, st = _tensor(q.in_types[1])
                        wd, wt = _tensor(q.in_types[2])
                        if maps[:3] == ["d0,d1", "d0", "d1"] and (sd, st, wd, wt) == ([M], "f32", [N], "f32") and \
                                q.ins[1:] == arg_names[2:4]:
                            epilogue = "requant"
                plan = dg.plan_matmul(fname, kind, epilogue, M, N, K, batch=batch, device_tensor_maps=device_tensor_maps,
                                      sm_count=sm_count)
                break
            if o.name == "linalg.generic" and _iterators(o.attrs) == ["parallel", "parallel", "reduction", "reduction"] \
                    and o.body == ["arith.extf", "arith.extf", "arith.mulf", "arith.addf"] and len(o.ins) == 2:
                deq = by_result.get(o.ins[1])
                if not deq or deq.name != "linalg.generic" or deq.body != ["arith.extsi", "arith.sitofp", "arith.mulf"] \
                        or "reduction" in _iterators(deq.attrs) or len(deq.ins) != 2:
                    continue
                (ad, at), (wd, wt), (sd, st) = _tensor(o.in_types[0]), _tensor(deq.in_types[0]), _tensor(deq.in_types[1])
                if (at, wt, st) != ("f16", "i4", "f16") or len(ad) != 3 or len(wd) != 3 or sd != wd[:2] or ad[1:] != wd[1:]:
                    continue
                if _maps(o.attrs, text) != ["d0,d2,d3", "d1,d2,d3", "d0,d1"] or not zero_fill(o.outs[0]):
                    continue
                t = consumer(o.result, ["arith.truncf"])
                if t is None or _tensor(t.result_type)[1] != "f16":
                    continue
                M, G, gs = ad
                N = wd[0]
                # the int4 tensor: a function argument, or bytes bitcast to i4 (two per byte)
                w_src = deq.ins[0]
                cast = by_result.get(w_src)
                if cast is not None:
                    if cast.name != "flow.tensor.bitcast":
                        continue
                    w_src = re.search(r"(%[\w.]+)", cast.attrs).group(1)
                if [o.ins[0], w_src, deq.ins[1]] != arg_names[:3]:
                    raise ValueError("@%s: expected arguments (activations, weights, scales)" % fname)
                plan = dg.plan_w4a16(fname, M, N, G * gs, group=gs, sm_count=sm_count)
                break
        if plan is not None:
            plans[fname] = plan
    return plans


# ---- the benchmark configurations as MLIR text ----------------------------------------------------------
_TRUNC = '''    %o = tensor.empty() : tensor<{shape}x{t}>
    %r = linalg.generic {{indexing_maps = [affine_map<({d}) -> ({d})>, affine_map<({d}) -> ({d})>],
                         iterator_types = [{par}]}}
        ins(%acc : tensor<{shape}xf32>) outs(%o : tensor<{shape}x{t}>) {{
      ^bb0(%in: f32, %out: {t}):
        %v = arith.truncf %in : f32 to {t}
        linalg.yield %v : {t}
    }} -> tensor<{shape}x{t}>
'''


def matmul_mlir(name: str, kind: str, epilogue: str, M: int, N: int, K: int, batch: int = 1) -> str:
    lead = "%dx" % batch if batch > 1 else ""
    acc_t = "i32" if kind == "i8" else "f32"
    zero = "0 : i32" if kind == "i8" else "0.000000e+00 : f32"
    op = "linalg.batch_matmul" if batch > 1 else "linalg.matmul"
    shape = "%s%dx%d" % (lead, M, N)
    out_t = {"acc": acc_t, "cast": kind, "requant": "f16"}[epilogue]
    args = "%%lhs: tensor<%s%dx%dx%s>, %%rhs: tensor<%s%dx%dx%s>" % (lead, M, K, kind, lead, K, N, kind)
    if epilogue == "requant":
        args += ", %%a_scale: tensor<%dxf32>, %%w_scale: tensor<%dxf32>" % (M, N)
    s = "  util.func public @%s(%s) -> tensor<%sx%s> {\n" % (name, args, shape, out_t)
    s += "    %%zero = arith.constant %s\n    %%e = tensor.empty() : tensor<%sx%s>\n" % (zero, shape, acc_t)
    s += "    %%fill = linalg.fill ins(%%zero : %s) outs(%%e : tensor<%sx%s>) -> tensor<%sx%s>\n" % (acc_t, shape, acc_t, shape, acc_t)
    s += "    %%acc = %s ins(%%lhs, %%rhs : tensor<%s%dx%dx%s>, tensor<%s%dx%dx%s>)\n" % (op, lead, M, K, kind, lead, K, N, kind)
    s += "        outs(%%fill : tensor<%sx%s>) -> tensor<%sx%s>\n" % (shape, acc_t, shape, acc_t)
    if epilogue == "cast":
        d = "d0, d1, d2" if batch > 1 else "d0, d1"
        par = ", ".join(['"parallel"'] * (3 if batch > 1 else 2))
        s += _TRUNC.format(shape=shape, t=kind, d=d, par=par)
        s += "    util.return %%r : tensor<%sx%s>\n  }\n" % (shape, kind)
    elif epilogue == "requant":
        s += "    %%o = tensor.empty() : tensor<%sxf16>\n" % shape
        s += ("    %%r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>,\n"
              "                                          affine_map<(d0, d1) -> (d1)>, affine_map<(d0, d1) -> (d0, d1)>],\n"
              "                         iterator_types = [\"parallel\", \"parallel\"]}\n"
              "        ins(%%acc, %%a_scale, %%w_scale : tensor<%sxi32>, tensor<%dxf32>, tensor<%dxf32>) outs(%%o : tensor<%sxf16>) {\n"
              "      ^bb0(%%in: i32, %%sa: f32, %%sw: f32, %%out: f16):\n"
              "        %%f = arith.sitofp %%in : i32 to f32\n"
              "        %%x = arith.mulf %%f, %%sa : f32\n"
              "        %%y = arith.mulf %%x, %%sw : f32\n"
              "        %%t = arith.truncf %%y : f32 to f16\n"
              "        linalg.yield %%t : f16\n"
              "    } -> tensor<%sxf16>\n" % (shape, M, N, shape, shape))
        s += "    util.return %%r : tensor<%sxf16>\n  }\n" % shape
    else:
        s += "    util.return %%acc : tensor<%sx%s>\n  }\n" % (shape, acc_t)
    return s


def w4a16_mlir(name: str, M: int, N: int, K: int, group: int = 128) -> str:
    G = K // group
    w3 = "%dx%dx%d" % (N, G, group)
    s = ("  util.func public @%s(%%a: tensor<%dx%dx%dxf16>, %%wq: tensor<%dx%dxi8>, %%scales: tensor<%dx%dxf16>) -> tensor<%dx%dxf16> {\n"
         % (name, M, G, group, N, K // 2, N, G, M, N))
    s += "    %%w4 = flow.tensor.bitcast %%wq : tensor<%dx%dxi8> -> tensor<%sxi4>\n" % (N, K // 2, w3)
    s += "    %%we = tensor.empty() : tensor<%sxf16>\n" % w3
    s += ("    %%deq = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2) -> (d0, d1, d2)>, affine_map<(d0, d1, d2) -> (d0, d1)>,\n"
          "                                            affine_map<(d0, d1, d2) -> (d0, d1, d2)>],\n"
          "                           iterator_types = [\"parallel\", \"parallel\", \"parallel\"]}\n"
          "        ins(%%w4, %%scales : tensor<%sxi4>, tensor<%dx%dxf16>) outs(%%we : tensor<%sxf16>) {\n"
          "      ^bb0(%%in: i4, %%s: f16, %%out: f16):\n"
          "        %%i = arith.extsi %%in : i4 to i32\n"
          "        %%f = arith.sitofp %%i : i32 to f16\n"
          "        %%d = arith.mulf %%f, %%s : f16\n"
          "        linalg.yield %%d : f16\n"
          "    } -> tensor<%sxf16>\n" % (w3, N, G, w3, w3))
    s += "    %%zero = arith.constant 0.000000e+00 : f32\n    %%e = tensor.empty() : tensor<%dx%dxf32>\n" % (M, N)
    s += "    %%fill = linalg.fill ins(%%zero : f32) outs(%%e : tensor<%dx%dxf32>) -> tensor<%dx%dxf32>\n" % (M, N, M, N)
    s += ("    %%acc = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2, d3) -> (d0, d2, d3)>, affine_map<(d0, d1, d2, d3) -> (d1, d2, d3)>,\n"
          "                                            affine_map<(d0, d1, d2, d3) -> (d0, d1)>],\n"
          "                           iterator_types = [\"parallel\", \"parallel\", \"reduction\", \"reduction\"]}\n"
          "        ins(%%a, %%deq : tensor<%dx%dx%dxf16>, tensor<%sxf16>) outs(%%fill : tensor<%dx%dxf32>) {\n"
          "      ^bb0(%%x: f16, %%w: f16, %%out: f32):\n"
          "        %%xe = arith.extf %%x : f16 to f32\n"
          "        %%we2 = arith.extf %%w : f16 to f32\n"
          "        %%p = arith.mulf %%xe, %%we2 : f32\n"
          "        %%sum = arith.addf %%p, %%out : f32\n"
          "        linalg.yield %%sum : f32\n"
          "    } -> tensor<%dx%dxf32>\n" % (M, G, group, w3, M, N, M, N))
    s += _TRUNC.format(shape="%dx%d" % (M, N), t="f16", d="d0, d1", par='"parallel", "parallel"')
    s += "    util.return %%r : tensor<%dx%dxf16>\n  }\n" % (M, N)
    return s


_HEADER = ('#cuda = #hal.device.target<"cuda", [#hal.executable.target<"cuda", "cuda-nvptx-fb", {}>]>\n'
           "module attributes {hal.device.targets = [#cuda]} {\n")


def config_mlir(config: str) -> str:
    """The benchmark configuration `config` ("c1" .. "c5") as a module of linalg-on-tensors functions,
    one function per shape of the configuration; function names are those of ``baseline_plans``."""
    body = ""
    if config == "c1":
        body += matmul_mlir("c1", "i8", "acc", 1024, 1024, 1024)
    elif config == "c2":
        body += matmul_mlir("c2", "f16", "cast", 4096, 4096, 4096)
        body += matmul_mlir("c2_bmm", "f16", "cast", 512, 512, 128, batch=32)
    elif config == "c3":
        for m in (1, 16, 512, 4096):
            body += matmul_mlir("c3_m%d" % m, "i8", "requant", m, 11008, 4096)
    elif config == "c4":
        for m in (1, 8, 16, 128, 2048):
            body += w4a16_mlir("c4_m%d" % m, m, 11008, 4096)
    elif config == "c5":
        for m in (16, 4096):
            body += w4a16_mlir("c5_m%d" % m, m, 28672, 8192)
    else:
        raise ValueError(config)
    return _HEADER + body + "}\n"


if __name__ == "__main__":
    import sys
    sys.stdout.write(config_mlir(sys.argv[1]))
