"""PTX pass of the CHECKED build: every global (or generic) load, store, atomic and reduction goes through a range test.

``compute-sanitizer`` is not always available where this library is tested, so the checked build variant
(``python -m vectorstorekit_b200.build --checked`` -> ``libvsk_cuda_checked.so``) instruments the kernels itself.
nvcc's own pipeline is run step by step (``build.py``); between the front end (PTX out) and ``ptxas`` this pass
rewrites each

    [@p] ld|st|atom|red[.volatile|.relaxed|...][.global] ... [%rdN+imm] ...

whose address is a register (addresses of module-level symbols are left alone) into

    {   add.s64 a, %rdN, imm
        a = vsk_chk_access(a, size | flags)      // csrc/checked.cuh, one copy per module
        the same instruction on [a]  }

``vsk_chk_access`` returns the address unchanged when it lies in a range the library knows (its own allocations with
the sizes the call asked for, plus buffers the caller announced) or is not a global address at all (shared and local
windows are bounded by the hardware); otherwise it records the first offending address and instruction size in the
device-side state and returns the address of a small sink buffer, so the access itself never leaves valid memory: no
trap, no fault, and the host reads the violation after the call.  Tensor-map (TMA) copies are bounds-checked by the
hardware against the extents in their descriptor and are not touched; the global side of an asynchronous
``cp.async`` copy is checked like a load.
"""
from __future__ import annotations

import re
import sys

_TYPE_BYTES = {"b8": 1, "u8": 1, "s8": 1, "b16": 2, "u16": 2, "s16": 2, "f16": 2, "bf16": 2, "b32": 4, "u32": 4,
               "s32": 4, "f32": 4, "f16x2": 4, "bf16x2": 4, "b64": 8, "u64": 8, "s64": 8, "f64": 8, "b128": 16}
_OTHER_SPACES = ("shared", "local", "param", "const")
_INSTR = re.compile(r"^(?P<indent>\s*)(?:@(?P<neg>!?)(?P<pred>%p\d+)\s+)?(?P<op>(?:ld|st|atom|red)\.[A-Za-z0-9_.:]+)(?P<rest>\s.*;.*)$")
# cp.async.{ca,cg}.shared.global [dst], [src], cp-size{, src-size};  - the global side is the SECOND address
_CPASYNC = re.compile(r"^(?P<indent>\s*)(?:@(?P<neg>!?)(?P<pred>%p\d+)\s+)?(?P<op>cp\.async\.c[ag]\.shared(?:::cta)?\.global[A-Za-z0-9_.:]*)"
                      r"(?P<head>\s+\[[^\]]+\]\s*,\s*)\[\s*(?P<base>%rd\d+)\s*(?:\+\s*(?P<imm>-?\d+))?\s*\](?P<tail>\s*,\s*(?P<size>\d+).*;.*)$")
_ADDR = re.compile(r"\[\s*(?P<base>%rd\d+)\s*(?:\+\s*(?P<imm>-?\d+))?\s*\]")
_CHECKER = re.compile(r"\.func\s*\(\.param\s+\.b64\s+\w+\)\s+(?P<name>_ZN\w*vsk_chk_access\w*)\s*\(")


def access_bytes(op: str) -> int:
    toks = op.split(".")
    vec = 1
    size = 0
    for t in toks:
        if t in ("v2", "v4", "v8"):
            vec = int(t[1])
        elif t in _TYPE_BYTES:
            size = _TYPE_BYTES[t]      # the last type token is the access type (atom.cas.b32, ld.global.nc.f32)
    return vec * size


def instrument(ptx: str) -> tuple[str, int]:
    m = _CHECKER.search(ptx)
    if not m:
        raise RuntimeError("the module does not define vsk_chk_access (is csrc/checked.cuh included?)")
    checker = m.group("name")
    out, sites = [], 0
    in_checker = False       # inside the checker's own declaration or body: it must not call itself
    depth = 0
    for line in ptx.split("\n"):
        if not in_checker and checker in line and ".func" in line:
            in_checker, depth = True, 0
        if in_checker:
            depth += line.count("{") - line.count("}")
            out.append(line)
            ends_decl = depth == 0 and line.rstrip().endswith(";") and "{" not in line     # forward declaration
            ends_body = depth == 0 and "}" in line
            if ends_decl or ends_body:
                in_checker = False
            continue
        mc = _CPASYNC.match(line)
        if mc:
            # asynchronous global -> shared copy: the source address goes through the checker (as a read of cp-size
            # bytes; a refused copy reads the sink instead)
            sites += 1
            ind, base, imm = mc.group("indent"), mc.group("base"), mc.group("imm") or "0"
            info = int(mc.group("size"))
            label = f"$L_vskc_{sites}"
            if mc.group("pred"):
                out.append(f"{ind}@{'' if mc.group('neg') else '!'}{mc.group('pred')} bra {label};")
            out.append(f"{ind}{{")
            out.append(f"{ind}.reg .b64 %vskc_a;")
            out.append(f"{ind}.param .b64 vskc_in;")
            out.append(f"{ind}.param .b32 vskc_sz;")
            out.append(f"{ind}.param .b64 vskc_out;")
            out.append(f"{ind}add.s64 %vskc_a, {base}, {imm};")
            out.append(f"{ind}st.param.b64 [vskc_in], %vskc_a;")
            out.append(f"{ind}st.param.b32 [vskc_sz], {info};")
            out.append(f"{ind}call.uni (vskc_out), {checker}, (vskc_in, vskc_sz);")
            out.append(f"{ind}ld.param.b64 %vskc_a, [vskc_out];")
            out.append(f"{ind}{mc.group('op')}{mc.group('head')}[%vskc_a]{mc.group('tail')}")
            out.append(f"{ind}}}")
            if mc.group("pred"):
                out.append(f"{label}:")
            continue
        mi = _INSTR.match(line)
        if not mi:
            out.append(line)
            continue
        op = mi.group("op")
        toks = op.split(".")
        if any(t.split("::")[0] in _OTHER_SPACES for t in toks):
            out.append(line)
            continue
        ma = _ADDR.search(mi.group("rest"))
        nbytes = access_bytes(op)
        if not ma or nbytes == 0:
            out.append(line)        # address of a module symbol, or nothing this pass understands
            continue
        sites += 1
        ind = mi.group("indent")
        base, imm = ma.group("base"), ma.group("imm") or "0"
        write = 0 if toks[0] == "ld" else 1
        info = nbytes | (write << 8)
        rest = mi.group("rest")
        new_rest = rest[:ma.start()] + "[%vskc_a]" + rest[ma.end():]
        label = f"$L_vskc_{sites}"
        if mi.group("pred"):
            # skip the whole block when the instruction's predicate is off
            out.append(f"{ind}@{'' if mi.group('neg') else '!'}{mi.group('pred')} bra {label};")
        out.append(f"{ind}{{")
        out.append(f"{ind}.reg .b64 %vskc_a;")
        out.append(f"{ind}.param .b64 vskc_in;")
        out.append(f"{ind}.param .b32 vskc_sz;")
        out.append(f"{ind}.param .b64 vskc_out;")
        out.append(f"{ind}add.s64 %vskc_a, {base}, {imm};")
        out.append(f"{ind}st.param.b64 [vskc_in], %vskc_a;")
        out.append(f"{ind}st.param.b32 [vskc_sz], {info};")
        out.append(f"{ind}call.uni (vskc_out), {checker}, (vskc_in, vskc_sz);")
        out.append(f"{ind}ld.param.b64 %vskc_a, [vskc_out];")
        out.append(f"{ind}{op}{new_rest}")
        out.append(f"{ind}}}")
        if mi.group("pred"):
            out.append(f"{label}:")
    return "\n".join(out), sites


def main(argv):
    path = argv[1]
    with open(path) as f:
        ptx = f.read()
    new, sites = instrument(ptx)
    with open(path, "w") as f:
        f.write(new)
    print(f"{path}: {sites} accesses instrumented")


if __name__ == "__main__":
    main(sys.argv)
