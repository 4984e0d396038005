"""Generates the binding file for an unmodified aiehlc example source.

aiehlc keeps host code and AIE kernels in one file; its compiler cuts every `__global__` kernel out, builds
it for the AIE and replaces the function name given to XAie_LoadElfMem by the embedded ELF
(src/llvm/aiehlc.cc:301-322, 469-607; src/preprocess/preporcess.py:8-23).  On B200 the example is compiled as
host code with `-D__global__=` (the kernel bodies become dead host functions whose ADDRESSES name the
kernels) and linked with a binding file that registers a CUDA launch under each of those addresses.  This
module writes that binding file:

  * a kernel whose body is the matmul loop nest of example/perf/aieml_perf.cc:72-82 or
    example/matrixmultiply/aieml_mm.cc:67-76 (`acc += a[i*N+k] * b[j*N+k]`, windows at fixed tile addresses or
    read through the AIE window API) is bound to the library's int32 matmul kernel with the tile size taken
    from the source's `#define N` -- with the golden loop's zero-initialised result, which is what the
    examples check against (aieml_mm.cc's own accumulator is never zeroed, :51,73);
  * a kernel in plain C that touches memory only through its two pointer parameters is re-emitted as a
    single-thread CUDA kernel with the same body (example/multi/multi_tile.cpp:39-47 and the like);
  * anything else (AIE vector API, fixed addresses outside a recognised pattern) is reported and left
    unbound, so XAie_LoadElfMem fails loudly for it.

    python -m aiehlc_b200.bindgen path/to/example.cc [-o binding.cu] [--host-out host.cc]

--host-out writes the example with its kernel bodies cut out, for sources whose kernels are not C++ the host
compiler accepts (example/matrixmultiply/aieml_mm.cc uses the AIE vector API).
"""
from __future__ import annotations

import argparse
import re
import sys
from dataclasses import dataclass, field
from pathlib import Path

DEFAULT_IN, DEFAULT_OUT = 0x1000, 0x6000
TILE_BASE = 0x70000          # data memory base the examples add to their window addresses (aieml_perf.cc:69-70)
PLAIN_WINDOW_BYTES = 4096    # output window reserved for a re-emitted plain-C kernel when no size hint is given


@dataclass
class Param:
    ctype: str
    name: str
    mem_address: int | None = None
    size_hint: int | None = None


@dataclass
class Kernel:
    name: str
    params: list[Param]
    body: str
    kind: str = "unsupported"      # "matmul" | "plain" | "unsupported"
    why: str = ""
    in_addr: int = DEFAULT_IN
    out_addr: int = DEFAULT_OUT
    n: int = 0                     # matmul: tile dimension
    defines: dict = field(default_factory=dict)


def _strip_comments(text: str) -> str:
    """Comments blanked out (same length, newlines kept), in source order: a `/*` inside a `//` comment or a
    string does not open a block comment."""
    out, i, n = [], 0, len(text)
    while i < n:
        c, nxt = text[i], text[i + 1] if i + 1 < n else ""
        if c == "/" and nxt == "/":
            j = text.find("\n", i)
            j = n if j < 0 else j
            out.append(" " * (j - i))
            i = j
        elif c == "/" and nxt == "*":
            j = text.find("*/", i + 2)
            j = n if j < 0 else j + 2
            out.append("".join(ch if ch == "\n" else " " for ch in text[i:j]))
            i = j
        elif c in "\"'":
            j = i + 1
            while j < n and text[j] != c:
                j += 2 if text[j] == "\\" else 1
            out.append(text[i:j + 1])
            i = j + 1
        else:
            out.append(c)
            i += 1
    return "".join(out)


def _match(text: str, start: int, open_ch: str, close_ch: str) -> int:
    """Index just past the bracket that closes the one at `start`."""
    depth = 0
    for i in range(start, len(text)):
        if text[i] == open_ch:
            depth += 1
        elif text[i] == close_ch:
            depth -= 1
            if depth == 0:
                return i + 1
    raise ValueError("unbalanced brackets in the source")


def _split_params(params: str) -> list[str]:
    out, depth, cur = [], 0, []
    for ch in params:
        if ch in "([":
            depth += 1
        elif ch in ")]":
            depth -= 1
        if ch == "," and depth == 0:
            out.append("".join(cur))
            cur = []
        else:
            cur.append(ch)
    if "".join(cur).strip():
        out.append("".join(cur))
    return out


def _parse_param(text: str) -> Param:
    addr = re.search(r"mem_address\s*:\s*(0x[0-9a-fA-F]+|\d+)", text)
    hint = re.search(r"size_hint\s*:\s*(\d+)", text)
    bare = re.sub(r"__attribute__\s*\(\(.*\)\)", "", text, flags=re.S).strip()
    m = re.match(r"(.*?)(\w+)\s*$", bare, flags=re.S)
    ctype, name = (m.group(1).strip(), m.group(2)) if m else (bare, "")
    return Param(ctype, name, int(addr.group(1), 0) if addr else None, int(hint.group(1)) if hint else None)


def parse_kernels(source: str) -> list[Kernel]:
    """Every `__global__ void name(params) { body }` of the source, classified."""
    text = _strip_comments(source)
    file_defines = {m.group(1): m.group(2) for m in re.finditer(r"^\s*#\s*define\s+(\w+)\s+(\S+)", text, flags=re.M)}
    kernels = []
    for m in re.finditer(r"__global__\s+void\s+(\w+)\s*\(", text):
        p_end = _match(text, m.end() - 1, "(", ")")
        b_start = text.index("{", p_end)
        b_end = _match(text, b_start, "{", "}")
        params = [_parse_param(p) for p in _split_params(text[m.end():p_end - 1])]
        k = Kernel(m.group(1), params, text[b_start:b_end], defines=dict(file_defines))
        k.defines.update({d.group(1): d.group(2)
                          for d in re.finditer(r"^\s*#\s*define\s+(\w+)\s+(\S+)", k.body, flags=re.M)})
        _classify(k)
        kernels.append(k)
    return kernels


_MATMUL = re.compile(r"(\w+)(?:\s*\[[^\]]*\])?\s*\+=\s*(\w+)\s*\[\s*(\w+)\s*\*\s*(\w+)\s*\+\s*(\w+)\s*\]\s*\*\s*"
                     r"(\w+)\s*\[\s*(\w+)\s*\*\s*(\w+)\s*\+\s*(\w+)\s*\]")
_ABS_PTR = re.compile(r"\(\s*\w[\w\s]*\*\s*\)\s*\(\s*(0x[0-9a-fA-F]+)\s*\+\s*(0x[0-9a-fA-F]+)\s*\)")


def _int_define(k: Kernel, name: str) -> int | None:
    v = k.defines.get(name)
    try:
        return int(v, 0) if v is not None else None
    except ValueError:
        return None


def _classify(k: Kernel) -> None:
    ins = [p for p in k.params if "out" not in p.name.lower() and "out" not in p.ctype.lower()]
    outs = [p for p in k.params if p not in ins]
    if ins and ins[0].mem_address is not None:
        k.in_addr = ins[0].mem_address
    if outs and outs[0].mem_address is not None:
        k.out_addr = outs[0].mem_address
    if outs and outs[0].mem_address is None and _int_define(k, "CORE_OP_MEM") is not None:
        k.out_addr = _int_define(k, "CORE_OP_MEM")
    if ins and ins[0].mem_address is None and _int_define(k, "CORE_IP_MEM") is not None:
        k.in_addr = _int_define(k, "CORE_IP_MEM")
    body = k.body
    mm = _MATMUL.search(body)
    if mm:
        _, _, i1, n1, k1, _, j2, n2, k2 = mm.groups()
        n = _int_define(k, n1)
        if n1 == n2 and k1 == k2 and i1 != j2 and n:
            k.kind, k.n = "matmul", n
            # windows given as fixed tile addresses: data memory base + window offset
            for base, off in _ABS_PTR.findall(body):
                if int(base, 0) == TILE_BASE:
                    decl = body[:body.index(off)].rsplit(";", 1)[-1]
                    if "out" in decl:
                        k.out_addr = int(off, 0)
                    elif "in" in decl:
                        k.in_addr = int(off, 0)
            return
    if re.search(r"\baie::|window_readincr|window_writeincr|chess_", body):
        k.why = "uses the AIE vector / window API outside a recognised pattern"
        return
    if _ABS_PTR.search(body) or re.search(r"\(\s*\w[\w\s]*\*\s*\)\s*0x[0-9a-fA-F]+", body):
        k.why = "addresses tile memory at fixed addresses outside a recognised pattern"
        return
    if len(k.params) != 2:
        k.why = "plain kernels are expected to take (in, out)"
        return
    if re.search(r"\bwhile\s*\(\s*(1|true)\s*\)|for\s*\(\s*;\s*;\s*\)", body):
        k.why = "does not terminate"
        return
    k.kind = "plain"


def host_source(source: str) -> str:
    """The example with every `__global__` kernel reduced to an empty function that keeps only the body's
    preprocessor lines (the examples define macros inside their kernels that the host code below uses):
    what is left compiles as plain host C++ whatever the kernel was written in.  The reference's own
    tool chain makes the same cut (src/preprocess/preporcess.py:8-23)."""
    text = _strip_comments(source)
    out, pos = [], 0
    for m in re.finditer(r"__global__\s+void\s+(\w+)\s*\(", text):
        p_end = _match(text, m.end() - 1, "(", ")")
        b_start = text.index("{", p_end)
        b_end = _match(text, b_start, "{", "}")
        keep = [ln for ln in source[b_start:b_end].splitlines() if ln.lstrip().startswith("#")]
        out.append(source[pos:b_start])
        out.append("{\n" + "\n".join(keep) + "\n}")
        pos = b_end
    out.append(source[pos:])
    return "".join(out)


def generate(source: str, origin: str = "the example") -> tuple[str, list[Kernel]]:
    """Binding file text for the kernels of `source`, and the kernels as classified."""
    kernels = parse_kernels(source)
    lines = [f"// Binding file generated by aiehlc_b200.bindgen for {origin} (compiled unmodified, -D__global__=).",
             '#include <cuda_runtime.h>', '', '#include "aiehlc_kernels.h"', '']
    for k in kernels:
        proto = ", ".join(p.ctype for p in k.params)
        if k.kind == "unsupported":
            lines += [f"// {k.name}: not bound ({k.why}); XAie_LoadElfMem reports an unknown kernel for it.", ""]
            continue
        lines.append(f"void {k.name}({proto});  // defined by the example; only its address is used")
        if k.kind == "matmul":
            lines += [f"static void __attribute__((constructor)) aiehlc_bind_{k.name}(void) {{",
                      f"  static const XAie_MmArgs args = {{{k.n}, {k.n}, {k.n}}};",
                      f'  XAie_KernelBind((const void*){k.name}, "{k.name}", (const void*)aiehlc_k_mm_i32, &args, sizeof args,',
                      f"                  {k.in_addr:#x}, {k.out_addr:#x}, 0);", "}", ""]
        else:
            cuda_params = ", ".join(f"{p.ctype} {p.name}" for p in k.params)
            out_p = next((p for p in k.params if "out" in p.name.lower()), k.params[-1])
            window = out_p.size_hint * 4 if out_p.size_hint else PLAIN_WINDOW_BYTES
            casts = ", ".join(f"({p.ctype})(info->{'out' if p is out_p else 'in'})" for p in k.params)
            lines += [f"__global__ void {k.name}_cuda({cuda_params}) {k.body}",
                      f"static int aiehlc_launch_{k.name}(const XAie_KernelLaunchInfo* info) {{",
                      f"  {k.name}_cuda<<<1, 1, 0, (cudaStream_t)info->stream>>>({casts});",
                      "  return (int)cudaGetLastError();", "}",
                      f"static void __attribute__((constructor)) aiehlc_bind_{k.name}(void) {{",
                      f'  XAie_KernelDesc d = {{"{k.name}", aiehlc_launch_{k.name}, 0, {window}, {k.in_addr:#x}, {k.out_addr:#x}, 0, 0, 0, 0}};',
                      f"  XAie_KernelRegister((const void*){k.name}, &d);", "}", ""]
    return "\n".join(lines), kernels


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("source")
    ap.add_argument("-o", "--output")
    ap.add_argument("--host-out", help="also write the example with its kernel bodies cut out (plain host C++)")
    args = ap.parse_args(argv)
    src = Path(args.source)
    text, kernels = generate(src.read_text(), origin=src.name)
    if args.host_out:
        Path(args.host_out).write_text(host_source(src.read_text()))
    if args.output:
        Path(args.output).write_text(text)
    else:
        sys.stdout.write(text)
    for k in kernels:
        what = {"matmul": f"int32 matmul {k.n}x{k.n}x{k.n}", "plain": "re-emitted as a CUDA kernel",
                "unsupported": f"NOT bound: {k.why}"}[k.kind]
        print(f"bindgen: {k.name}: {what} (in {k.in_addr:#x}, out {k.out_addr:#x})", file=sys.stderr)
    return 0 if any(k.kind != "unsupported" for k in kernels) else 1


if __name__ == "__main__":
    sys.exit(main())
