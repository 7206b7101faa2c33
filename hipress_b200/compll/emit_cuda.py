"""CompLL back end: one DSL function -> sm_100a CUDA source.

Where the reference emits a chain of thrust calls with host round trips (two
synchronising ``thrust::reduce``, a ``thrust::transform`` with one thread per
output byte, four host-to-device header copies per tensor:
src/CompLL/GCGen/output/TernGradEncode/TernGradEncode_body.h:115-123 of
mark14wu/hipress; rules at src/CompLL/GCGen/tree.py:197-288), this emitter
produces

* one *reduction kernel* that evaluates every ``reduce`` of the function in a
  single pass (warp shuffles, per-block partials, the last block finishes), and
* one *map kernel* per ``map`` statement that recomputes the scalar expressions
  from the reduced values, packs sub-byte outputs LSB-first (the order the DSL's
  ``V[i]`` subscript reads them back), and writes the ``concat`` header fields
  from the device -- no host synchronisation anywhere.

``random<float>(lo, hi)`` draws from Philox4x32-7 keyed by (seed, element index,
call site), so every element gets an independent, reproducible number (the
reference seeds an LCG identically in every thread, output/naive_random.hpp).
"""
from __future__ import annotations

from dataclasses import dataclass

from . import frontend as F
from .frontend import CompileError

C_TYPES = {"float": "float", "int": "int32_t", "uint": "uint32_t", "uint8": "uint8_t",
           "uint1": "uint8_t", "uint2": "uint8_t", "uint4": "uint8_t"}
SIZEOF = {"float": 4, "int": 4, "uint": 4, "uint8": 1, "uint1": 1, "uint2": 1, "uint4": 1}
CALLS = {"floor": "floorf", "ceil": "ceilf", "abs": "fabsf", "sqrt": "sqrtf", "min": "fminf",
         "max": "fmaxf", "exp": "expf", "log": "logf", "round": "rintf"}
BUILTIN_REDUCERS = {"smaller": "fminf({a}, {b})", "greater": "fmaxf({a}, {b})", "sum": "({a} + {b})"}


@dataclass
class Sym:
    name: str
    kind: str               # param_scalar | param_vector | reduced | derived | extracted | lambda | vector
    type: F.Type
    expr: object = None     # init expression (derived / reduced)
    slot: int = -1          # reduced: index into the scalar buffer
    bits: object = None     # sub-byte vectors: bit width expression
    alias: tuple = None     # local vector: (base param name, byte offset)
    count: object = None    # local vector: element count expression
    header_off: int = -1    # extracted scalar: byte offset in the source buffer


class Emitter:
    def __init__(self, fn: F.Function):
        self.fn = fn
        self.syms: dict[str, Sym] = {}
        self.order: list[str] = []      # scalar symbols in evaluation order
        self.reduces: list[Sym] = []
        self.maps: list[tuple] = []     # (target vector name, Map expr)
        self.concats: list[tuple] = []  # (target param, [(kind, name, offset)], vector name or None)
        self.extracts: list = []
        self.rand_sites = 0
        self.stages: list = []          # ('reduce', [Sym]) | ('map', index into self.maps), source order
        self._analyse()

    # ------------------------------------------------------------ analysis
    def _add(self, s: Sym):
        if s.name in self.syms:
            raise CompileError(f"redefinition of {s.name}")
        self.syms[s.name] = s
        return s

    def _analyse(self):
        fn = self.fn
        for ty, name in fn.params:
            self._add(Sym(name, "param_vector" if ty.vector else "param_scalar", ty))
        for st in fn.body:
            if isinstance(st, F.Decl):
                self._decl(st)
            elif isinstance(st, F.Assign):
                self._assign(st)
            elif isinstance(st, F.ExprStmt) and isinstance(st.value, F.Extract):
                self._extract(st.value)
            elif isinstance(st, F.Return):
                continue
            else:
                raise CompileError(f"statement not supported at function scope: {type(st).__name__}")

    def _decl(self, st: F.Decl):
        ty, init = st.type, st.init
        if ty.name == "lambda_func":
            if not isinstance(init, F.Lambda):
                raise CompileError(f"lambda_func {st.name} needs a lambda", st.line)
            self._add(Sym(st.name, "lambda", ty, init))
            return
        if ty.vector:
            s = self._add(Sym(st.name, "vector", ty, bits=self._bits_of(ty)))
            if isinstance(init, F.Map):
                s.count = init.count if init.count is not None else F.SizeOf(init.vec)
                self.maps.append((st.name, init))
                self.stages.append(("map", len(self.maps) - 1))
                self.order.append(st.name)
            elif init is not None:
                raise CompileError(f"vector {st.name}: only map(...) can initialise a vector", st.line)
            return
        if isinstance(init, F.Reduce):
            s = self._add(Sym(st.name, "reduced", ty, init, slot=len(self.reduces)))
            self.reduces.append(s)
            self._stage_reduce(s)
        elif init is None:
            self._add(Sym(st.name, "extracted", ty))
        else:
            self._add(Sym(st.name, "derived", ty, init))
        self.order.append(st.name)

    def _assign(self, st: F.Assign):
        if not isinstance(st.target, F.Name):
            raise CompileError("assignment target must be a name", st.line)
        name = st.target.id
        tgt = self.syms.get(name)
        if tgt is None:
            raise CompileError(f"assignment to undeclared {name}", st.line)
        v = st.value
        if isinstance(v, F.Map):
            if tgt.kind not in ("param_vector", "vector"):
                raise CompileError(f"map result must go to a vector, {name} is not one", st.line)
            if tgt.kind == "vector":
                tgt.count = v.count if v.count is not None else F.SizeOf(v.vec)
                if name not in self.order:
                    self.order.append(name)
            self.maps.append((name, v))
            self.stages.append(("map", len(self.maps) - 1))
        elif isinstance(v, F.Call) and v.fn in ("topk", "scatter", "scatter_add"):
            # library-lowered stages: exact top-k selection / sparse scatter of the
            # run-time library (radix select in shared memory, block compaction)
            if tgt.kind != "param_vector":
                raise CompileError(f"{v.fn} needs a vector parameter on the left", st.line)
            if v.fn == "topk":
                if len(v.args) not in (2, 3) or not all(isinstance(x, F.Name) for x in
                                                          (v.args[0],) + tuple(v.args[2:])):
                    raise CompileError("topk(vector, k[, companion]) takes vector names", st.line)
            elif len(v.args) != 2 or not isinstance(v.args[0], F.Name):
                raise CompileError(f"{v.fn}(payload, scale) takes a payload vector and a scale", st.line)
            # scatter overwrites the target (zero, then place); scatter_add merges into it
            self.stages.append(("topk" if v.fn == "topk" else "scatter", name, v))
        elif isinstance(v, F.Concat):
            if tgt.kind != "param_vector":
                raise CompileError("the left-hand side of concat must be a function parameter", st.line)
            self._concat(name, v)
        elif isinstance(v, F.Reduce):
            tgt.kind, tgt.expr, tgt.slot = "reduced", v, len(self.reduces)
            self.reduces.append(tgt)
            self._stage_reduce(tgt)
        elif tgt.kind in ("extracted", "derived"):
            tgt.kind, tgt.expr = "derived", v
        else:
            raise CompileError(f"cannot assign to {name}", st.line)

    def _stage_reduce(self, s: Sym):
        """Adjacent reduces share one pass over the data."""
        if self.stages and self.stages[-1][0] == "reduce":
            self.stages[-1][1].append(s)
        else:
            self.stages.append(("reduce", [s]))

    def _bits_of(self, ty: F.Type):
        if ty.bits is not None:
            return ty.bits
        if ty.name in ("uint1", "uint2", "uint4"):
            return F.Num(str(F.BASIC_BITS[ty.name]), False)
        return None

    def _concat(self, target: str, c: F.Concat):
        off, fields, vec = 0, [], None
        for i, p in enumerate(c.parts):
            if not isinstance(p, F.Name) or p.id not in self.syms:
                raise CompileError("concat arguments must be declared names")
            s = self.syms[p.id]
            if s.kind == "vector":
                if i != len(c.parts) - 1:
                    raise CompileError("a vector may only be the last argument of concat")
                s.alias = (target, off)
                vec = s.name
            else:
                fields.append((s.name, off))
                off += SIZEOF[s.type.name]
        self.concats.append((target, fields, vec))

    def _extract(self, e: F.Extract):
        if not isinstance(e.src, F.Name) or self.syms.get(e.src.id, Sym("", "", None)).kind != "param_vector":
            raise CompileError("extract source must be a vector parameter")
        off = 0
        for i, t in enumerate(e.targets):
            s = self.syms.get(t)
            if s is None:
                raise CompileError(f"extract target {t} is not declared")
            if s.kind == "vector":
                if i != len(e.targets) - 1:
                    raise CompileError("a vector may only be the last target of extract")
                s.alias = (e.src.id, off)
                # element count = remaining bytes * 8 / bits
                s.count = ("extract", e.src.id, off)
                self.order.append(s.name)
            else:
                s.kind, s.header_off, s.alias = "extracted", off, (e.src.id, off)
                off += SIZEOF[s.type.name]
        self.extracts.append(e)

    # ------------------------------------------------------- expressions
    def expr(self, e, local: set, ctx: str = "c.") -> str:
        """C expression for `e`.  Names in `local` are lambda locals/parameters."""
        X = lambda x: self.expr(x, local, ctx)  # noqa: E731
        if isinstance(e, F.Num):
            return (e.text + ("f" if "." in e.text or "e" in e.text.lower() else ".0f")) if e.is_float \
                else e.text
        if isinstance(e, F.Name):
            if e.id in local:
                return f"l_{e.id}"
            s = self.syms.get(e.id)
            if s is None:
                raise CompileError(f"undeclared name {e.id}")
            return f"{ctx}v_{e.id}"
        if isinstance(e, F.Unary):
            return f"({e.op}{X(e.x)})"
        if isinstance(e, F.Binary):
            if e.op == "%":
                return f"({X(e.a)} % {X(e.b)})"
            return f"({X(e.a)} {e.op} {X(e.b)})"
        if isinstance(e, F.Ternary):
            return f"({X(e.c)} ? {X(e.a)} : {X(e.b)})"
        if isinstance(e, F.Call):
            fn = CALLS.get(e.fn)
            if fn is None:
                if e.fn in self.syms and self.syms[e.fn].kind == "lambda":
                    return f"fn_{e.fn}(c, {', '.join(X(a) for a in e.args)})"
                raise CompileError(f"unknown function {e.fn}")
            return f"{fn}({', '.join(X(a) for a in e.args)})"
        if isinstance(e, F.SizeOf):
            if not isinstance(e.base, F.Name):
                raise CompileError(".size needs a vector name")
            return f"{ctx}n_{e.base.id}"
        if isinstance(e, F.Index):
            if not isinstance(e.base, F.Name):
                raise CompileError("only named vectors can be subscripted")
            s = self.syms.get(e.base.id)
            if s is None or s.kind not in ("param_vector", "vector"):
                raise CompileError(f"{e.base.id} is not a vector")
            hook = getattr(self, "_index_hook", None)
            if hook is not None:      # fused target: the element at the own index lives in a register
                got = hook(s, e.idx, local)
                if got is not None:
                    return got
            i = X(e.idx)
            if s.bits is not None:
                b = self.expr(s.bits, set(), ctx)
                return (f"compll_get_bits({ctx}v_{s.name}, (uint64_t)({i}), (uint32_t)({b}))")
            return f"{ctx}v_{s.name}[{i}]"
        if isinstance(e, F.Random):
            site = self.rand_sites
            self.rand_sites += 1
            hook = getattr(self, "_random_hook", None)
            if hook is not None:      # fused target: one Philox call serves four elements
                return f"({X(e.lo)} + ({X(e.hi)} - {X(e.lo)}) * {hook(site)})"
            return (f"({X(e.lo)} + ({X(e.hi)} - {X(e.lo)}) * "
                    f"compll_rand01(c.seed, (uint64_t)l_{self._counter}, {site}u))")
        raise CompileError(f"expression not supported here: {type(e).__name__}")

    # ---------------------------------------------------------- lambdas
    def stmts(self, body, local: set, ret_partial: bool, indent="  ") -> str:
        out = []
        for st in body:
            if isinstance(st, F.Decl):
                local.add(st.name)
                init = f" = {self.expr(st.init, local)}" if st.init is not None else ""
                out.append(f"{indent}{C_TYPES[st.type.name]} l_{st.name}{init};")
            elif isinstance(st, F.Assign):
                out.append(f"{indent}{self.expr(st.target, local)} = {self.expr(st.value, local)};")
            elif isinstance(st, F.If):
                out.append(f"{indent}if ({self.expr(st.cond, local)}) {{")
                out.append(self.stmts(st.then, set(local), ret_partial, indent + "  "))
                if st.other:
                    out.append(f"{indent}}} else {{")
                    out.append(self.stmts(st.other, set(local), ret_partial, indent + "  "))
                out.append(f"{indent}}}")
            elif isinstance(st, F.Return):
                rv = getattr(self, "_return_to", None)
                if rv is not None:    # inlined lambda: the caller wraps the body in do { } while (0)
                    out.append(f"{indent}{{ {rv} = {self.expr(st.value, local)}; break; }}")
                else:
                    out.append(f"{indent}return {self.expr(st.value, local)};")
            elif isinstance(st, F.ExprStmt):
                out.append(f"{indent}{self.expr(st.value, local)};")
            else:
                raise CompileError(f"statement not supported in a lambda: {type(st).__name__}")
        return "\n".join(out)

    def lambda_fn(self, s: Sym, qual: str = "__device__ __forceinline__") -> str:
        lam: F.Lambda = s.expr
        local = {n for _, n in lam.params}
        self._counter = lam.params[0][1] if lam.params else "zero"
        ret = "uint32_t" if lam.ret.is_subbyte() else C_TYPES[lam.ret.name]
        params = ", ".join(f"{C_TYPES[t.name]} l_{n}" for t, n in lam.params)
        body = self.stmts(lam.body, local, lam.ret.is_subbyte())
        return (f"{qual} {ret} fn_{s.name}(const Ctx& c"
                f"{', ' if params else ''}{params}) {{\n{body}\n}}\n")

    # ---------------------------------------------------------- pieces
    def ctx_struct(self) -> str:
        rows = ["struct Ctx {", "  uint64_t seed;"]
        for s in self.syms.values():
            if s.kind in ("param_scalar", "reduced", "derived", "extracted"):
                rows.append(f"  {C_TYPES[s.type.name]} v_{s.name};")
            elif s.kind == "param_vector":
                rows.append(f"  {C_TYPES[s.type.name]}* v_{s.name};\n  uint64_t n_{s.name};")
            elif s.kind == "vector":
                rows.append(f"  uint8_t* v_{s.name};\n  uint64_t n_{s.name};" if s.bits is not None
                            else f"  {C_TYPES[s.type.name]}* v_{s.name};\n  uint64_t n_{s.name};")
        rows.append("};")
        return "\n".join(rows)

    def kernel_params(self) -> str:
        ps = []
        for ty, name in self.fn.params:
            if ty.vector:
                ps += [f"{C_TYPES[ty.name]}* p_{name}", f"uint64_t n_{name}"]
            else:
                ps.append(f"{C_TYPES[ty.name]} p_{name}")
        ps += ["float* scalars", "uint64_t seed"]
        return ", ".join(ps)

    def kernel_args(self) -> str:
        a = []
        for ty, name in self.fn.params:
            a += [f"p_{name}", f"n_{name}"] if ty.vector else [f"p_{name}"]
        return ", ".join(a + ["scalars", "seed"])

    def prologue(self, upto_reduced_only=False) -> str:
        """Builds Ctx c: parameters, extracted header fields, reduced values and the
        derived scalars in source order."""
        rows = ["  Ctx c;", "  c.seed = seed;"]
        for ty, name in self.fn.params:
            rows.append(f"  c.v_{name} = p_{name};")
            if ty.vector:
                rows.append(f"  c.n_{name} = n_{name};")
        for name in self.order:
            s = self.syms[name]
            if s.kind == "extracted":
                base, off = s.alias
                rows.append(f"  c.v_{name} = compll_load<{C_TYPES[s.type.name]}>("
                            f"reinterpret_cast<const uint8_t*>(p_{base}) + {off});")
            elif s.kind == "reduced":
                if upto_reduced_only:
                    continue
                rows.append(f"  c.v_{name} = ({C_TYPES[s.type.name]})scalars[{s.slot}];")
            elif s.kind == "derived":
                if upto_reduced_only and self._depends_on_reduced(s.expr):
                    continue
                rows.append(f"  c.v_{name} = ({C_TYPES[s.type.name]})({self.expr(s.expr, set())});")
            elif s.kind == "vector":  # a local vector is an alias into a parameter buffer
                if s.alias is None:
                    raise CompileError(f"vector {s.name} is never placed with concat or extract")
                base, off = s.alias
                ptr = f"reinterpret_cast<uint8_t*>(p_{base}) + {off}"
                if s.bits is None:
                    rows.append(f"  c.v_{s.name} = reinterpret_cast<{C_TYPES[s.type.name]}*>({ptr});")
                else:
                    rows.append(f"  c.v_{s.name} = {ptr};")
                if isinstance(s.count, tuple):  # extracted: remaining bytes * 8 / bits
                    bexp = self.expr(s.bits, set()) if s.bits is not None else str(8 * SIZEOF[s.type.name])
                    rows.append(f"  c.n_{s.name} = (n_{base} * sizeof(*p_{base}) - {off}) * 8 / "
                                f"(uint64_t)({bexp});")
                elif not upto_reduced_only or not self._depends_on_reduced(s.count):
                    rows.append(f"  c.n_{s.name} = (uint64_t)({self.expr(s.count, set())});")
        return "\n".join(rows)

    def _depends_on_extracted(self, e) -> bool:
        if isinstance(e, F.Name):
            sy = self.syms.get(e.id)
            if sy is None:
                return False
            if sy.kind == "extracted":
                return True
            return sy.kind == "derived" and self._depends_on_extracted(sy.expr)
        if not isinstance(e, F.Expr):
            return False
        for f in getattr(e, "__dataclass_fields__", {}):
            v = getattr(e, f)
            if isinstance(v, F.Expr) and self._depends_on_extracted(v):
                return True
            if isinstance(v, list) and any(isinstance(a, F.Expr) and self._depends_on_extracted(a) for a in v):
                return True
        return False

    def _depends_on_reduced(self, e) -> bool:
        if isinstance(e, F.Name):
            s = self.syms.get(e.id)
            if s is None:
                return False
            if s.kind == "reduced":
                return True
            return s.kind == "derived" and self._depends_on_reduced(s.expr)
        if isinstance(e, (F.Num, type(None))):
            return False
        if isinstance(e, tuple):
            return False
        return any(self._depends_on_reduced(getattr(e, f)) for f in getattr(e, "__dataclass_fields__", {})
                   if isinstance(getattr(e, f), F.Expr)) or any(
            self._depends_on_reduced(a) for f in getattr(e, "__dataclass_fields__", {})
            if isinstance(getattr(e, f), list) for a in getattr(e, f) if isinstance(a, F.Expr))

    # ---------------------------------------------------------- kernels
    def reduce_kernel(self, gi: int, group: list) -> str:
        name = self.fn.name
        nred = len(group)
        init, step, comb, fin = [], [], [], []
        n_expr = None
        for k, s in enumerate(group):
            r: F.Reduce = s.expr
            if not isinstance(r.vec, F.Name):
                raise CompileError("reduce needs a vector name")
            vec = r.vec.id
            n_expr = n_expr or f"n_{vec}"
            ty = C_TYPES[s.type.name]
            init.append(f"  {ty} acc{k} = ({ty})({self.expr(r.init, set())});")
            step.append(f"    if (i < n_{vec}) acc{k} = {self._apply(r.fn, f'acc{k}', f'({ty})p_{vec}[i]')};")
            comb.append(f"    {{ {ty} o = __shfl_xor_sync(0xffffffffu, acc{k}, off); "
                        f"acc{k} = {self._apply(r.fn, f'acc{k}', 'o')}; }}")
        body = f"""
__global__ void __launch_bounds__(256) {name}_reduce{gi}_kernel({self.kernel_params()}, float* partials,
                                                           unsigned int* ticket) {{
{self.prologue(upto_reduced_only=True)}
{chr(10).join(init)}
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < {n_expr}; i += stride) {{
{chr(10).join(step)}
  }}
  for (int off = 16; off > 0; off >>= 1) {{
{chr(10).join(comb)}
  }}
  __shared__ float sh[{nred}][8];
  __shared__ bool last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {{ {' '.join(f'sh[{k}][warp] = (float)acc{k};' for k in range(nred))} }}
  __syncthreads();
  if (threadIdx.x == 0) {{
{self._fold(group, 'sh[{k}][{w}]', 8, 'partials[{k} * gridDim.x + blockIdx.x]')}
    __threadfence();
    last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }}
  __syncthreads();
  if (last && threadIdx.x == 0) {{
    __threadfence();
{self._fold(group, '__ldcg(&partials[{k} * gridDim.x + {w}])', 'gridDim.x', 'scalars[{slot}]')}
    *ticket = 0;
  }}
}}
"""
        return body

    def _fold(self, group, src, count, dst) -> str:
        rows = []
        for k, s in enumerate(group):
            r: F.Reduce = s.expr
            ty = C_TYPES[s.type.name]
            rows.append(f"    {{ {ty} a = ({ty}){src.format(k=k, w=0)}; for (unsigned w = 1; w < {count}; ++w) "
                        f"a = {self._apply(r.fn, 'a', '(' + ty + ')' + src.format(k=k, w='w'))}; "
                        f"{dst.format(k=k, slot=s.slot)} = (float)a; }}")
        return "\n".join(rows)

    def _apply(self, fn, a, b) -> str:
        if isinstance(fn, F.Name) and fn.id in BUILTIN_REDUCERS and fn.id not in self.syms:
            return BUILTIN_REDUCERS[fn.id].format(a=a, b=b)
        if isinstance(fn, F.Name) and fn.id in self.syms and self.syms[fn.id].kind == "lambda":
            return f"fn_{fn.id}(c, {a}, {b})"
        raise CompileError("the third argument of reduce must be a lambda or smaller/greater/sum")

    def map_kernel(self, idx: int, target: str, m: F.Map, write_header: bool) -> str:
        name = self.fn.name
        tgt = self.syms[target]
        if not isinstance(m.fn, F.Name) or self.syms.get(m.fn.id, Sym("", "", None)).kind != "lambda":
            raise CompileError("the second argument of map must be a lambda")
        lam_sym = self.syms[m.fn.id]
        lam: F.Lambda = lam_sym.expr
        if m.vec is not None:
            if not isinstance(m.vec, F.Name):
                raise CompileError("map over a vector needs a vector name")
            count = f"c.n_{m.vec.id}"
            arg = lambda i: f"c.v_{m.vec.id}[{i}]"  # noqa: E731
        else:
            count = f"(uint64_t)({self.expr(m.count, set())})"
            arg = lambda i: f"({C_TYPES[lam.params[0][0].name]})({i})"  # noqa: E731
        header = ""
        if write_header:
            rows = []
            for tname, fields, _ in self.concats:
                for fname, off in fields:
                    s = self.syms[fname]
                    rows.append(f"    compll_store<{C_TYPES[s.type.name]}>(reinterpret_cast<uint8_t*>"
                                f"(p_{tname}) + {off}, c.v_{fname});")
            if rows:
                header = "  if (blockIdx.x == 0 && threadIdx.x == 0) {\n" + "\n".join(rows) + "\n  }\n"
        if tgt.bits is not None:
            bits = self.expr(tgt.bits, set())
            body = f"""  const uint32_t bits = (uint32_t)({bits});
  const uint32_t per = 8u / bits, mask = (1u << bits) - 1u;
  const uint64_t count = {count};
  const uint64_t nbytes = (count + per - 1) / per;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < nbytes; b += stride) {{
    uint32_t byte = 0;
    for (uint32_t e = 0; e < per; ++e) {{
      const uint64_t i = b * per + e;
      if (i < count) byte |= ((uint32_t)fn_{lam_sym.name}(c, {arg('i')}) & mask) << (e * bits);
    }}
    c.v_{target}[b] = (uint8_t)byte;
  }}"""
        else:
            body = f"""  const uint64_t count = {count};
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride)
    c.v_{target}[i] = fn_{lam_sym.name}(c, {arg('i')});"""
        return f"""
__global__ void __launch_bounds__(256) {name}_map{idx}_kernel({self.kernel_params()}) {{
{self.prologue()}
{header}{body}
}}
"""

    # ------------------------------------------------------------- files
    def body_source(self) -> str:
        """The generated kernels (``-b``)."""
        name = self.fn.name
        self.rand_sites = 0  # call sites are numbered per emission: both targets agree
        lambdas = "\n".join(self.lambda_fn(s) for s in self.syms.values() if s.kind == "lambda")
        fused = self.fused_plan()
        if fused is not None:
            # one persistent kernel for the whole function (emit_fused.py); the random
            # call sites are numbered as the staged kernels and the CPU target number them
            from .emit_fused import FusedGen
            self.rand_sites = 0
            maps, reduces = FusedGen(fused).kernel_source(), ""
        else:
            # staged target; runs of maps between library calls may still share a kernel
            segs = self.segments()
            in_seg = {self.stages[k][1] for i0, cnt, _ in segs for k in range(i0, i0 + cnt)}
            last_map = len(self.maps) - 1
            maps = "\n".join(self.map_kernel(i, t, m, i == last_map)
                             for i, (t, m) in enumerate(self.maps) if i not in in_seg)
            if segs:
                from .emit_fused import FusedGen
                for si, (i0, cnt, plan) in enumerate(segs):
                    has_last = any(self.stages[k][1] == last_map for k in range(i0, i0 + cnt))
                    maps += FusedGen(plan, tag=f"seg{si}", write_header=has_last).kernel_source()
            reduces = "\n".join(self.reduce_kernel(gi, st[1]) for gi, st in enumerate(self.stages)
                                if st[0] == "reduce")
        src_comment = "\n".join("//   " + l for l in self.fn.source.strip().splitlines())
        return f"""// Generated by hipress_b200.compll from the DSL function {name}:
//
{src_comment}
//
// Do not edit; regenerate with  python -m hipress_b200.compll <file>.pse -b -w -r -f torch
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "hipress/compll_rt.cuh"

namespace compll_gen_{name} {{

{self.ctx_struct()}

{lambdas}
{reduces}
{maps}
}}  // namespace compll_gen_{name}
"""

    def fused_plan(self):
        """The one-launch plan of this function, or None when it keeps one kernel per
        stage (library-lowered stages, lambdas calling lambdas; ``fuse=False``)."""
        if not getattr(self, "fuse", True):
            return None
        if not hasattr(self, "_fused_plan"):
            from .emit_fused import FusedPlan
            plan = FusedPlan(self)
            self._fused_plan = plan if plan.ok else None
        return self._fused_plan

    def segments(self):
        """Fusable runs of maps of a function that keeps the staged target (see
        emit_fused.fused_segments); empty when the whole function is one launch."""
        if not getattr(self, "fuse", True) or self.fused_plan() is not None:
            return []
        if not hasattr(self, "_segments"):
            from .emit_fused import fused_segments
            self._segments = fused_segments(self)
        return self._segments

    def wrapper_source(self) -> str:
        """``extern "C"`` launcher (``-w``): stream-ordered, no host synchronisation."""
        name = self.fn.name
        ps = []
        for ty, pname in self.fn.params:
            if ty.vector:
                ps += [f"{C_TYPES[ty.name]}* p_{pname}", f"uint64_t n_{pname}"]
            else:
                ps.append(f"{C_TYPES[ty.name]} p_{pname}")
        sig = ", ".join(ps + ["void* scratch", "uint64_t seed", "void* stream"])
        nred = len(self.reduces)
        n_main = None
        for ty, pname in self.fn.params:
            if ty.vector:
                n_main = n_main or f"n_{pname}"
        rows = []
        uses_lib = any(st[0] in ("topk", "scatter") for st in self.stages)
        if uses_lib:
            rows.append("  compll_gen_%s::Ctx h;  // host copy of the parameters for library calls" % name)
            for ty, pname in self.fn.params:
                rows.append(f"  h.v_{pname} = p_{pname};")
                if ty.vector:
                    rows.append(f"  h.n_{pname} = n_{pname};")
            for sname in self.order:
                sy = self.syms[sname]
                if sy.kind == "derived" and not self._depends_on_reduced(sy.expr) and \
                        not self._depends_on_extracted(sy.expr):
                    rows.append(f"  h.v_{sname} = ({C_TYPES[sy.type.name]})({self.expr(sy.expr, set(), 'h.')});")
        seg_at = {i0: (si, cnt, plan) for si, (i0, cnt, plan) in enumerate(self.segments())}
        skip = 0
        for gi, st in enumerate(self.stages):
            if skip:
                skip -= 1
                continue
            if gi in seg_at:
                from .emit_fused import FusedGen
                si, cnt, plan = seg_at[gi]
                rows.append(FusedGen(plan, tag=f"seg{si}").launch_rows())
                skip = cnt - 1
                continue
            if st[0] == "topk":
                _, target, call = st
                vec = call.args[0].id
                comp = call.args[2].id if len(call.args) == 3 else None
                kexp = self.expr(call.args[1], set(), "h.")
                rows.append(f"""  {{
    const uint64_t k = (uint64_t)({kexp});
    if (k < 1 || k > n_{vec}) return -1;
    if (n_{target} < hp_sparse_payload_bytes(k)) return -2;
    int rc = hp_cuda_sparse_encode({4 if comp else 5}, nullptr, p_{vec}, {('p_' + comp) if comp else 'nullptr'}, n_{vec}, k, k, 0.0f, 0,
                                   reinterpret_cast<uint8_t*>(p_{target}),
                                   reinterpret_cast<uint8_t*>(scratch) + (kScalarBytes / 256 * 256 + 256), kLibScratch, 0, stream);
    if (rc) return rc;
  }}""")
                continue
            if st[0] == "scatter":
                _, target, call = st
                src = call.args[0].id
                sexp = self.expr(call.args[1], set(), "h.")
                rows.append(f"""  {{
    if (n_{src} < 16) return -1;
    const uint64_t kmax = (n_{src} - 16) / 8;   // capacity of the payload buffer in pairs
    int rc = hp_cuda_sparse_decode(reinterpret_cast<const uint8_t*>(p_{src}), p_{target}, n_{target},
                                   kmax, (float)({sexp}), {1 if call.fn == "scatter_add" else 0}, stream);
    if (rc) return rc;
  }}""")
                continue
            if st[0] == "reduce":
                rows.append(f"  compll_gen_{name}::{name}_reduce{gi}_kernel<<<grid, 256, 0, st>>>"
                            f"({self.kernel_args()}, partials, ticket);")
            else:
                rows.append(f"  compll_gen_{name}::{name}_map{st[1]}_kernel<<<grid, 256, 0, st>>>"
                            f"({self.kernel_args()});")
        if self.fused_plan() is not None:
            from .emit_fused import FusedGen
            rows = [FusedGen(self.fused_plan()).launch_rows()]
        red = f"""  float* partials = scalars + 16;
  unsigned int* ticket = reinterpret_cast<unsigned int*>(scalars + 16 + {max(nred, 1)} * kMaxBlocks);
  (void)partials; (void)ticket;
"""
        launches = "\n".join(rows)
        lib_decl = ""
        if uses_lib:
            lib_decl = """
// run-time library entry points (libhipress_cuda.so)
extern "C" int hp_cuda_sparse_encode(int alg, const float* g, float* a, float* u, uint64_t n, uint64_t k,
                                     uint64_t kmax, float momentum, int update, uint8_t* out,
                                     void* workspace, uint64_t workspace_bytes, int max_ctas, void* stream);
extern "C" int hp_cuda_sparse_decode(const uint8_t* payload, float* out, uint64_t n, uint64_t kmax,
                                     float scale, int accumulate, void* stream);
static inline uint64_t hp_sparse_payload_bytes(uint64_t k) { return 16 + 2 * ((4 * k + 15) / 16 * 16); }
"""
        return f"""// Generated by hipress_b200.compll: launcher of {name}.
#include "{name}_body.cuh"
{lib_decl}
namespace {{
constexpr int kMaxBlocks = 1184;  // 148 SMs x 8
constexpr uint64_t kScalarBytes = (16 + {max(nred, 1)} * kMaxBlocks + 4) * sizeof(float) + 240;
constexpr uint64_t kLibScratch = {'(49216 + (8ull << 20))' if uses_lib else '0'};  // radix histograms + candidate list
}}

extern "C" {{

// bytes of device scratch the launcher needs (zero-initialised once by the caller)
uint64_t compll_{name}_scratch_bytes() {{ return kScalarBytes / 256 * 256 + 256 + kLibScratch; }}

int compll_{name}({sig}) {{
  cudaStream_t st = (cudaStream_t)stream;
  float* scalars = static_cast<float*>(scratch);
  uint64_t work = {n_main};
  int grid = (int)((work + 255) / 256);
  if (grid < 1) grid = 1;
  if (grid > kMaxBlocks) grid = kMaxBlocks;
{red}{launches}
  return (int)cudaGetLastError();
}}

}}  // extern "C"
"""

    @property
    def uses_library(self) -> bool:
        return any(st[0] in ("topk", "scatter") for st in self.stages)

    def host_source(self) -> str:
        """The CPU target: the same function as sequential C++ (``-t cpu``)."""
        from .emit_host import host_source
        return host_source(self)

    def register_source(self, framework: str = "torch") -> str:
        """Python registration (``-r -f torch``): binds the launcher to torch tensors."""
        name = self.fn.name
        if framework != "torch":
            raise CompileError(f"unsupported target framework {framework!r}: this generator emits "
                               "PyTorch bindings (-f torch)")
        args, conv, ctypes_sig = [], [], []
        for ty, pname in self.fn.params:
            args.append(pname)
            if ty.vector:
                conv.append(f"{pname}.data_ptr(), {pname}.numel()")
                ctypes_sig += ["C.c_void_p", "C.c_uint64"]
            else:
                conv.append(f"{pname}")
                ctypes_sig.append({"float": "C.c_float", "int": "C.c_int32", "uint": "C.c_uint32"}
                                  .get(ty.name, "C.c_uint8"))
        vecs = [pname for ty, pname in self.fn.params if ty.vector]
        return f'''"""Generated by hipress_b200.compll: PyTorch binding of {name}.  Tensors on the
CPU run the generated C++ (lib{name}_cpu.so), CUDA tensors the sm_100a kernels
(lib{name}.so)."""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None
_cpu = None
_scratch = {{}}
_SIG = [{", ".join(ctypes_sig)}]


def _load():
    global _lib
    if _lib is None:
        _lib = C.CDLL(os.path.join(_HERE, "lib{name}.so"))
        _lib.compll_{name}.restype = C.c_int
        _lib.compll_{name}.argtypes = _SIG + [C.c_void_p, C.c_uint64, C.c_void_p]
        _lib.compll_{name}_scratch_bytes.restype = C.c_uint64
    return _lib


def _load_cpu():
    global _cpu
    if _cpu is None:
        _cpu = C.CDLL(os.path.join(_HERE, "lib{name}_cpu.so"))
        _cpu.compll_{name}_cpu.restype = C.c_int
        _cpu.compll_{name}_cpu.argtypes = _SIG + [C.c_uint64]
    return _cpu


def {name}({", ".join(args)}, seed=0, stream=None):
    """In-place op: vectors are contiguous torch tensors allocated by the caller,
    all on one device."""
    vectors = ({", ".join(vecs)},)
    if any(not t.is_contiguous() for t in vectors):
        raise ValueError("{name}: tensors must be contiguous")
    if len({{t.device for t in vectors}}) != 1:
        raise ValueError("{name}: tensors must share one device")
    if not vectors[0].is_cuda:
        rc = _load_cpu().compll_{name}_cpu({", ".join(conv)}, seed)
        if rc != 0:
            raise RuntimeError(f"{name}: error {{rc}}")
        return
    lib = _load()
    dev = vectors[0].device.index
    with torch.cuda.device(dev):
        if dev not in _scratch:
            _scratch[dev] = torch.zeros(int(lib.compll_{name}_scratch_bytes()), dtype=torch.uint8,
                                        device="cuda")
        st = (stream or torch.cuda.current_stream()).cuda_stream
        rc = lib.compll_{name}({", ".join(conv)}, _scratch[dev].data_ptr(), seed, st)
    if rc != 0:
        raise RuntimeError(f"{name}: CUDA error {{rc}}")
'''


def generate(src: str, fuse: bool = True) -> Emitter:
    """``fuse=False`` keeps one kernel per reduce group / map (the staged target)."""
    em = Emitter(F.parse(src))
    em.fuse = fuse
    return em
