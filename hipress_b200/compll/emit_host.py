"""CompLL back end, CPU target: one DSL function -> plain sequential C++.

The reference registers every generated operator for the CPU as well as the GPU
(``FCompute<cpu>`` with ``thrust::host``: src/CompLL/GCGen/unit.py:231-272 and
output/TernGradEncode/TernGradEncode.cc:26-28 of mark14wu/hipress).  This target
plays that part: it reuses the analysis, the lambdas and the context struct of
the CUDA emitter and replaces each kernel by a loop, so a DSL function can be run
and tested without a GPU.  Quantisation, bit packing, header layout and the random
numbers (Philox keyed by seed, element, call site) are those of the CUDA target;
a ``reduce`` folds left to right here and as a tree there, so a floating-point
``sum`` may differ in the last bits while ``min`` / ``max`` agree exactly.
"""
from __future__ import annotations

from . import frontend as F
from .emit_cuda import C_TYPES, CompileError, Emitter, Sym


def _reduce_stage(em: Emitter, group: list) -> str:
    init, step, fin = [], [], []
    n_expr = None
    for k, s in enumerate(group):
        r: F.Reduce = s.expr
        if not isinstance(r.vec, F.Name):
            raise CompileError("reduce needs a vector name")
        vec = r.vec.id
        n_expr = n_expr or f"n_{vec}"
        ty = C_TYPES[s.type.name]
        init.append(f"    {ty} acc{k} = ({ty})({em.expr(r.init, set())});")
        step.append(f"      if (i < n_{vec}) acc{k} = {em._apply(r.fn, f'acc{k}', f'({ty})p_{vec}[i]')};")
        fin.append(f"    scalars[{s.slot}] = (float)acc{k};")
    nl = "\n"
    return f"""  {{  // reduce
{_indent(em.prologue(upto_reduced_only=True))}
{nl.join(init)}
    for (uint64_t i = 0; i < {n_expr}; ++i) {{
{nl.join(step)}
    }}
{nl.join(fin)}
  }}"""


def _indent(text: str, by: str = "  ") -> str:
    return "\n".join(by + row if row else row for row in text.splitlines())


def _map_stage(em: Emitter, target: str, m: F.Map, write_header: bool) -> str:
    tgt = em.syms[target]
    if not isinstance(m.fn, F.Name) or em.syms.get(m.fn.id, Sym("", "", None)).kind != "lambda":
        raise CompileError("the second argument of map must be a lambda")
    lam_sym = em.syms[m.fn.id]
    lam: F.Lambda = lam_sym.expr
    if m.vec is not None:
        if not isinstance(m.vec, F.Name):
            raise CompileError("map over a vector needs a vector name")
        count = f"c.n_{m.vec.id}"
        arg = f"c.v_{m.vec.id}[i]"
    else:
        count = f"(uint64_t)({em.expr(m.count, set())})"
        arg = f"({C_TYPES[lam.params[0][0].name]})(i)"
    header = []
    if write_header:
        for tname, fields, _ in em.concats:
            for fname, off in fields:
                s = em.syms[fname]
                header.append(f"    compll_store<{C_TYPES[s.type.name]}>(reinterpret_cast<uint8_t*>"
                              f"(p_{tname}) + {off}, c.v_{fname});")
    if tgt.bits is not None:
        body = f"""    const uint32_t bits = (uint32_t)({em.expr(tgt.bits, set())});
    const uint32_t per = 8u / bits, mask = (1u << bits) - 1u;
    const uint64_t count = {count};
    const uint64_t nbytes = (count + per - 1) / per;
    for (uint64_t b = 0; b < nbytes; ++b) {{
      uint32_t byte = 0;
      for (uint32_t e = 0; e < per; ++e) {{
        const uint64_t i = b * per + e;
        if (i < count) byte |= ((uint32_t)fn_{lam_sym.name}(c, {arg}) & mask) << (e * bits);
      }}
      c.v_{target}[b] = (uint8_t)byte;
    }}"""
    else:
        body = f"""    const uint64_t count = {count};
    for (uint64_t i = 0; i < count; ++i) c.v_{target}[i] = fn_{lam_sym.name}(c, {arg});"""
    nl = "\n"
    return f"""  {{  // map -> {target}
{_indent(em.prologue())}
{nl.join(header)}
{body}
  }}"""


def _library_stage(em: Emitter, st) -> str:
    if st[0] == "topk":
        _, target, call = st
        vec = call.args[0].id
        comp = call.args[2].id if len(call.args) == 3 else None
        kexp = em.expr(call.args[1], set(), "h.")
        return f"""  {{  // topk -> {target}
    const uint64_t k = (uint64_t)({kexp});
    if (k < 1 || k > n_{vec}) return -1;
    if (n_{target} < hp_sparse_payload_bytes(k)) return -2;
    int rc = hp_cpu_sparse_select({4 if comp else 5}, p_{vec}, {('p_' + comp) if comp else 'nullptr'}, n_{vec}, k,
                                  reinterpret_cast<uint8_t*>(p_{target}), k);
    if (rc) return rc;
  }}"""
    _, target, call = st
    src = call.args[0].id
    sexp = em.expr(call.args[1], set(), "h.")
    return f"""  {{  // scatter -> {target}
    if (n_{src} < 16) return -1;
    const uint64_t kmax = (n_{src} - 16) / 8;   // capacity of the payload buffer in pairs
    int rc = hp_cpu_sparse_decode(reinterpret_cast<const uint8_t*>(p_{src}), p_{target}, n_{target},
                                  kmax, (float)({sexp}), {1 if call.fn == "scatter_add" else 0});
    if (rc) return rc;
  }}"""


def host_source(em: Emitter) -> str:
    name = em.fn.name
    em.rand_sites = 0  # same call-site numbers as the CUDA target
    lambdas = "\n".join(em.lambda_fn(s, "static inline") for s in em.syms.values() if s.kind == "lambda")
    ps = []
    for ty, pname in em.fn.params:
        if ty.vector:
            ps += [f"{C_TYPES[ty.name]}* p_{pname}", f"uint64_t n_{pname}"]
        else:
            ps.append(f"{C_TYPES[ty.name]} p_{pname}")
    sig = ", ".join(ps + ["uint64_t seed"])
    rows = []
    if em.uses_library:
        rows.append("  Ctx h;  // parameters and the scalars that depend on nothing computed, for library calls")
        for ty, pname in em.fn.params:
            rows.append(f"  h.v_{pname} = p_{pname};")
            if ty.vector:
                rows.append(f"  h.n_{pname} = n_{pname};")
        for sname in em.order:
            sy = em.syms[sname]
            if sy.kind == "derived" and not em._depends_on_reduced(sy.expr) and \
                    not em._depends_on_extracted(sy.expr):
                rows.append(f"  h.v_{sname} = ({C_TYPES[sy.type.name]})({em.expr(sy.expr, set(), 'h.')});")
    for st in em.stages:
        if st[0] == "reduce":
            rows.append(_reduce_stage(em, st[1]))
        elif st[0] == "map":
            target, m = em.maps[st[1]]
            rows.append(_map_stage(em, target, m, st[1] == len(em.maps) - 1))
        else:
            rows.append(_library_stage(em, st))
    lib_decl = ""
    if em.uses_library:
        lib_decl = """
// run-time library entry points (libhipress_cpu.so)
extern "C" int hp_cpu_sparse_select(int alg, float* v, float* u, uint64_t n, uint64_t k, uint8_t* out,
                                    uint64_t kmax);
extern "C" int hp_cpu_sparse_decode(const uint8_t* payload, float* out, uint64_t n, uint64_t kmax,
                                    float scale, int accumulate);
static inline uint64_t hp_sparse_payload_bytes(uint64_t k) { return 16 + 2 * ((4 * k + 15) / 16 * 16); }
"""
    src_comment = "\n".join("//   " + row for row in em.fn.source.strip().splitlines())
    body = "\n".join(rows)
    return f"""// Generated by hipress_b200.compll from the DSL function {name} (CPU target):
//
{src_comment}
//
// Do not edit; regenerate with  python -m hipress_b200.compll <file>.pse -t cpu
#include <math.h>
#include <stdint.h>
#include "hipress/compll_rt.cuh"
{lib_decl}
namespace compll_host_{name} {{

{em.ctx_struct()}

{lambdas}
}}  // namespace compll_host_{name}

extern "C" int compll_{name}_cpu({sig}) {{
  using namespace compll_host_{name};
  float scalars[{max(len(em.reduces), 1)}] = {{0}};
  (void)scalars; (void)seed;
{body}
  return 0;
}}
"""
