"""Extract the reference's own known-answer tests into JSON fixtures.

Reads (as text — nothing of the reference is built or run) the `#[cfg(test)]` modules of the reference's
op backends, `runtime/src/providers/cuda/backend/<op>.rs`, which are written with the `OpTest` helper
(runtime/src/testing.rs), e.g.

    let out = OpTest::new(Op::Gather)
        .input([3, 4], vec![1.0f32, 2.0, ...])
        .input([2], vec![0i32, 2])
        .attr("axis", AttributeType::Int(1))
        .output([3, 2])
        .run::<f32>()
        .unwrap();
    assert_eq!(out, vec![2.0, 4.0, ...]);

and writes one JSON file per op under tests/golden/kats/ with, per test function, the feeds, attributes,
declared output shape, expected values (exact or with the test's epsilon) or the expected error
substring.  Also copies the byte content of the ORT-CPU attention goldens
(runtime/tests/fixtures/attention_{q,k,v,out}.f32, 8 little-endian f32 each) into attention.json.

Only literal data is understood: `vec![..]`, `vec![x; n]`, ranges mapped to floats, `.map(f16::from_f32)`
and simple `let` bindings of those.  Test functions that compute their expectation with host code, or
chain the output of one OpTest into another, are listed in kats/_skipped.json with the reason; a few of
them are restated by hand in tests/test_reference_kats.py.

Usage:  python tests/golden/extract_kats.py [/path/to/reference]
"""
from __future__ import annotations

import json
import os
import re
import struct
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "kats")

SUFFIX = re.compile(r"(?<![A-Za-z_])(-?\d[\d_]*(?:\.[\d_]*)?(?:[eE][+-]?\d+)?)_?(f16|f32|f64|i8|u8|i16|u16|i32|u32|i64|u64|usize|isize)\b")
TYPE_OF_SUFFIX = {"f16": "float16", "f32": "float32", "f64": "float64", "i8": "int8", "u8": "uint8", "i16": "int16",
                  "u16": "uint16", "i32": "int32", "u32": "uint32", "i64": "int64", "u64": "uint64"}
RUST_TYPE = dict(TYPE_OF_SUFFIX, bool="bool")


def match_paren(s: str, i: int, open_="(", close=")") -> int:
    """Index of the bracket closing the one at s[i]."""
    depth = 0
    in_str = False
    j = i
    while j < len(s):
        ch = s[j]
        if in_str:
            if ch == "\\":
                j += 1
            elif ch == '"':
                in_str = False
        elif ch == '"':
            in_str = True
        elif ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
            if depth == 0:
                return j
        j += 1
    raise ValueError("unbalanced")


def split_top(s: str, sep=","):
    parts, depth, cur, in_str = [], 0, "", False
    for ch in s:
        if in_str:
            cur += ch
            if ch == '"':
                in_str = False
            continue
        if ch == '"':
            in_str = True
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == sep and depth == 0:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        parts.append(cur)
    return [p.strip() for p in parts]


class Unsupported(Exception):
    pass


def eval_data(expr: str, env: dict):
    """Evaluate a Rust data literal.  Returns (python list | scalar, dtype name or None)."""
    e = expr.strip()
    if e.startswith("&"):
        e = e[1:].strip()
    if e in env:
        return env[e]
    m = re.fullmatch(r"(\w+)\.clone\(\)", e)
    if m and m.group(1) in env:
        return env[m.group(1)]
    dtype = None
    m = re.fullmatch(r"Vec::<(\w+)>::new\(\)", e)
    if m:
        return [], RUST_TYPE.get(m.group(1))
    m = re.fullmatch(r"\((-?\d+)\.\.(=?)(-?\d+)\)\s*\.map\(\|(\w+)\|\s*\4 as (\w+)\)\s*\.collect(?:::<[^>]*>)?\(\)", e)
    if m:
        lo, incl, hi, _, ty = m.groups()
        vals = list(range(int(lo), int(hi) + (1 if incl else 0)))
        return ([float(v) for v in vals] if ty.startswith("f") else vals), RUST_TYPE.get(ty)
    m = re.fullmatch(r"\[(.*)\]\s*\.map\(f16::from_f32\)(?:\s*\.to_vec\(\))?", e, re.S)
    if m:
        vals, _ = eval_data("vec![" + m.group(1) + "]", env)
        return vals, "float16"
    if e.startswith("vec!["):
        inner = e[5:match_paren(e, 4)]
    elif e.startswith("["):
        inner = e[1:match_paren(e, 0)]
    else:
        raise Unsupported(f"data expression `{e[:60]}`")
    rep = split_top(inner, ";")
    if len(rep) == 2:
        v, dt = eval_scalar(rep[0])
        n = eval_int(rep[1])
        return [v] * n, dt
    vals = []
    for item in split_top(inner):
        v, dt = eval_scalar(item)
        vals.append(v)
        dtype = dtype or dt
    return vals, dtype


MODULE_CONSTS = {}


def eval_int(e: str) -> int:
    e = SUFFIX.sub(r"\1", e.strip())
    for k, v in MODULE_CONSTS.items():
        e = re.sub(r"\b%s\b" % k, str(v), e)
    if not re.fullmatch(r"[\d\s*+\-()_]+", e):
        raise Unsupported(f"int expression `{e}`")
    return int(eval(e.replace("_", "")))


CONSTS = {"f32::MAX": (3.4028234663852886e38, "float32"), "f32::MIN": (-3.4028234663852886e38, "float32"),
          "f32::INFINITY": (float("inf"), "float32"), "f32::NEG_INFINITY": (float("-inf"), "float32"),
          "f32::NAN": (float("nan"), "float32"), "i64::MAX": (2 ** 63 - 1, "int64"), "i64::MIN": (-(2 ** 63), "int64"),
          "i32::MAX": (2 ** 31 - 1, "int32"), "i32::MIN": (-(2 ** 31), "int32"), "true": (True, "bool"), "false": (False, "bool")}


def eval_scalar(item: str):
    s = item.strip()
    if s in CONSTS:
        return CONSTS[s]
    m = re.fullmatch(r"f16::from_f32\((.*)\)", s)
    if m:
        v, _ = eval_scalar(m.group(1))
        return float(v), "float16"
    m = SUFFIX.fullmatch(s)
    if m:
        num, ty = m.group(1).replace("_", ""), m.group(2)
        return (float(num) if ty.startswith("f") else int(num)), TYPE_OF_SUFFIX.get(ty)
    if re.fullmatch(r"-?\d[\d_]*", s):
        return int(s.replace("_", "")), None
    if re.fullmatch(r"-?\d[\d_]*\.[\d_]*(?:[eE][+-]?\d+)?|-?\d+[eE][+-]?\d+", s):
        return float(s.replace("_", "")), None
    raise Unsupported(f"scalar `{s[:40]}`")


def eval_dims(e: str):
    e = e.strip()
    if e.startswith("&"):
        e = e[1:]
    if not e.startswith("["):
        raise Unsupported(f"dims `{e}`")
    inner = e[1:match_paren(e, 0)]
    return [eval_int(x) for x in split_top(inner)] if inner.strip() else []


def parse_attr(val: str):
    m = re.fullmatch(r"AttributeType::(\w+)\((.*)\)", val.strip(), re.S)
    if not m:
        raise Unsupported(f"attribute `{val[:60]}`")
    kind, body = m.group(1), m.group(2).strip()
    if kind == "Int":
        return {"kind": "int", "value": eval_int(body)}
    if kind == "Ints":
        vals, _ = eval_data(body, {})
        return {"kind": "ints", "value": [int(v) for v in vals]}
    if kind == "Float":
        return {"kind": "float", "value": float(eval_scalar(body)[0])}
    if kind == "String":
        mm = re.search(r'"([^"]*)"', body)
        if not mm:
            raise Unsupported("string attribute")
        return {"kind": "string", "value": mm.group(1)}
    if kind == "Tensor":
        mm = re.fullmatch(r"Tensor::from_vec\((.*)\)(?:\s*\.(?:unwrap|expect)\([^)]*\))?", body, re.S)
        if mm:
            args = split_top(mm.group(1))
            dims = eval_dims(args[0]) if args[0].strip().startswith(("[", "&[")) else [int(v) for v in eval_data(args[0], {})[0]]
            vals, dt = eval_data(args[1], {})
            return {"kind": "tensor", "dims": dims, "dtype": dt, "value": vals}
    raise Unsupported(f"attribute kind {kind}")


def parse_chain(src: str, start: int, env: dict):
    """Parse `OpTest::new(Op::X).a(..).b(..)` starting at `start`; returns (case dict, end index)."""
    m = re.compile(r"OpTest::new\(Op::(\w+)\)").match(src, start)
    case = {"op": m.group(1), "feeds": [], "attrs": {}, "output": None, "run": None}
    i = m.end()
    while True:
        mm = re.compile(r"\s*\.(\w+)(?:::<([^>]*)>)?\(").match(src, i)
        if not mm:
            break
        name, generic = mm.group(1), mm.group(2)
        close = match_paren(src, mm.end() - 1)
        args = src[mm.end():close]
        i = close + 1
        if name in ("input", "constant"):
            a = split_top(args)
            dims = eval_dims(a[0])
            vals, dt = eval_data(",".join(a[1:]), env)
            case["feeds"].append({"kind": name, "dims": dims, "dtype": dt, "data": vals})
        elif name == "attr":
            a = split_top(args)
            key = re.search(r'"([^"]*)"', a[0]).group(1)
            case["attrs"][key] = parse_attr(",".join(a[1:]))
        elif name == "output":
            case["output"] = eval_dims(args)
        elif name == "run":
            case["run"] = RUST_TYPE.get(generic, generic)
        elif name == "run_err":
            case["run"] = "err"
        elif name in ("unwrap", "expect"):
            continue
        else:
            raise Unsupported(f"OpTest method .{name}")
    return case, i


def finish_dtypes(case):
    """Untyped literals take the dtype of a typed sibling (Rust infers the Vec's element type)."""
    for f in case["feeds"]:
        if f["dtype"] is None:
            if any(isinstance(v, float) for v in f["data"]):
                f["dtype"] = "float32" if case.get("run") in (None, "err", "float32", "bool") else case["run"]
            else:
                raise Unsupported("feed without a dtype suffix")
        if f["dtype"] == "bool":
            f["data"] = [bool(v) for v in f["data"]]


def sanitize(v):
    if isinstance(v, float):
        if v != v:
            return "nan"
        if v in (float("inf"), float("-inf")):
            return "inf" if v > 0 else "-inf"
    return v


def parse_test_fn(name: str, body: str):
    env = {}
    for m in re.finditer(r"let\s+(?:mut\s+)?(\w+)(?:\s*:\s*[^=]+?)?\s*=\s*", body):
        var = m.group(1)
        j = m.end()
        # find the terminating ';' at depth 0
        depth, k, in_str = 0, j, False
        while k < len(body):
            ch = body[k]
            if in_str:
                if ch == '"':
                    in_str = False
            elif ch == '"':
                in_str = True
            elif ch in "([{":
                depth += 1
            elif ch in ")]}":
                depth -= 1
            elif ch == ";" and depth == 0:
                break
            k += 1
        expr = body[j:k].strip()
        if expr.startswith("OpTest::new"):
            continue
        try:
            env[var] = eval_data(expr, env)
        except (Unsupported, ValueError, SyntaxError):
            pass
    chains = [m.start() for m in re.finditer(r"OpTest::new\(", body)]
    if len(chains) != 1:
        raise Unsupported(f"{len(chains)} OpTest chains in one test")
    case, end = parse_chain(body, chains[0], env)
    finish_dtypes(case)
    rest = body[end:]
    if case["run"] == "err":
        mm = re.search(r'contains\("([^"]+)"\)', rest)
        case["expect"] = {"kind": "error", "contains": mm.group(1) if mm else "unsupported"}
    else:
        mm = re.search(r"assert_eq!\(\s*out\s*,", rest)
        mc = re.search(r"assert_close(_eps)?\(\s*&out\s*,", rest)
        if mm:
            close = match_paren(rest, rest.index("(", mm.start()))
            args = split_top(rest[rest.index("(", mm.start()) + 1:close])
            vals, _ = eval_data(args[1], env)
            case["expect"] = {"kind": "eq", "values": vals}
        elif mc:
            close = match_paren(rest, rest.index("(", mc.start()))
            args = split_top(rest[rest.index("(", mc.start()) + 1:close])
            vals, _ = eval_data(args[1], env)
            eps = float(eval_scalar(args[2])[0]) if mc.group(1) else 1.1920929e-07  # approx's default epsilon for f32
            case["expect"] = {"kind": "close", "values": vals, "eps": eps}
        else:
            raise Unsupported("no recognised assertion on `out`")
        case["expect"]["values"] = [sanitize(v) for v in case["expect"]["values"]]
    for f in case["feeds"]:
        f["data"] = [sanitize(v) for v in f["data"]]
    case["name"] = name
    return case


def test_functions(src: str):
    for m in re.finditer(r"#\[test\](?:\s*#\[[^\]]*\])*\s*fn\s+(\w+)\s*\(\s*\)\s*\{", src):
        ignored = "#[ignore" in src[m.start():m.end()]
        close = match_paren(src, m.end() - 1)
        yield m.group(1), src[m.end():close], ignored, src.count("\n", 0, m.start()) + 1


# backends of CNN ops and of shape-only ops whose attribute forms this build does not take: no fixtures are written
OUTSIDE_THE_OPERATOR_PATH = {"conv.rs", "max_pool.rs", "global_average_pool.rs", "constant.rs"}


def main(ref):
    backend = os.path.join(ref, "runtime/src/providers/cuda/backend")
    os.makedirs(OUT, exist_ok=True)
    skipped = {}
    total = 0
    for fn in sorted(os.listdir(backend)):
        if not fn.endswith(".rs") or fn in OUTSIDE_THE_OPERATOR_PATH:
            continue
        src = open(os.path.join(backend, fn)).read()
        if "OpTest" not in src:
            continue
        cases = []
        MODULE_CONSTS.clear()
        for mc in re.finditer(r"const\s+(\w+)\s*:\s*(?:i32|i64|usize)\s*=\s*(-?\d+)\s*;", src):
            MODULE_CONSTS[mc.group(1)] = int(mc.group(2))
        for name, body, ignored, line in test_functions(src):
            if "OpTest::new" not in body:
                continue
            try:
                case = parse_test_fn(name, body)
                case["source"] = f"runtime/src/providers/cuda/backend/{fn}:{line}"
                case["ignored_in_reference"] = ignored
                cases.append(case)
            except (Unsupported, ValueError, KeyError, IndexError, AttributeError) as e:
                skipped[f"{fn}::{name}"] = str(e)
        if cases:
            with open(os.path.join(OUT, fn[:-3] + ".json"), "w") as f:
                json.dump(cases, f, indent=1)
            total += len(cases)
    fx = os.path.join(ref, "runtime/tests/fixtures")
    att = {"source": "runtime/tests/fixtures/attention_{q,k,v,out}.f32 (ORT-CPU goldens; graph in runtime/tests/graphs/attention.rs:9-56)"}
    for k in ("q", "k", "v", "out"):
        raw = open(os.path.join(fx, f"attention_{k}.f32"), "rb").read()
        att[k] = list(struct.unpack("<%df" % (len(raw) // 4), raw))
    with open(os.path.join(OUT, "attention.json"), "w") as f:
        json.dump(att, f, indent=1)
    with open(os.path.join(OUT, "_skipped.json"), "w") as f:
        json.dump(skipped, f, indent=1, sort_keys=True)
    print(f"extracted {total} cases, skipped {len(skipped)}")
    for k, v in sorted(skipped.items()):
        print("  skipped", k, "-", v)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/extract_kats.py /path/to/the/reference/checkout")
    main(sys.argv[1])
