"""CompLL back end, fused CUDA target: ONE launch per DSL function.

The stage-by-stage target (emit_cuda.py) turns every ``reduce`` group and every
``map`` into a kernel of its own, so ``TbqEncode`` (three maps) crossed HBM three
times.  This module plans the same function as a sequence of *phases* and emits
one persistent kernel that runs them back to back:

* consecutive ``map`` / ``reduce`` stages over the same index range join one phase
  when every value they take from a vector written earlier in the phase is the
  element at their own index; that element is then forwarded in a register, each
  input is loaded once (128-bit loads, four consecutive elements per thread) and
  only the last value written to a vector is stored;
* a stage that needs the *result* of a reduction of the current phase, reads a
  freshly written vector at another index, or covers another range starts a new
  phase behind a grid barrier (cooperative launch; the barrier is bounded);
* a ``reduce`` accumulates while its phase streams by: per-thread partial, warp
  shuffle, one partial per block; behind the barrier every block folds the
  partials (no second kernel, no host round trip);
* sub-byte results (``uint<b>``) are packed at warp level: a thread builds the
  4*b-bit fragment of its four elements and ``__shfl_down_sync`` assembles whole
  32-bit words, which the owning lanes store;
* ``random<float>`` costs one Philox call per four elements.

Functions with library-lowered stages (``topk``, ``scatter``) keep the staged
target for those stages; a run of maps between them still becomes one kernel
(``fused_segments``: DgcEncode's two state updates are one pass).  The rules this replaces: one ``thrust::transform`` per map with one
thread per output byte and a serial pack loop (src/CompLL/GCGen/tree.py:197-244,
unit.py:469-482 of mark14wu/hipress).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from . import frontend as F
from .emit_cuda import C_TYPES, SIZEOF, CompileError, Emitter, Sym


def _walk(e):
    """Every expression node below (and including) e, statements included."""
    if isinstance(e, list):
        for x in e:
            yield from _walk(x)
        return
    if e is None or isinstance(e, (str, int, float, bool, F.Type, tuple)):
        return
    yield e
    for f in getattr(e, "__dataclass_fields__", {}):
        v = getattr(e, f)
        if isinstance(v, (F.Expr, list)) or hasattr(v, "__dataclass_fields__"):
            yield from _walk(v)


@dataclass
class Item:
    kind: str                 # "map" | "reduce"
    target: str = ""          # map: vector written
    m: object = None          # map: F.Map
    sym: Sym = None           # reduce: the reduced symbol
    index: int = -1           # map: index into em.maps


@dataclass
class Phase:
    count: str                # C expression of the element count
    items: list = field(default_factory=list)
    written: list = field(default_factory=list)      # vectors written, in order
    reduced: set = field(default_factory=set)        # reduced symbols produced here
    read_elsewhere: set = field(default_factory=set)  # vectors read at an index other than the own one


class FusedPlan:
    """Phase plan of one function; ``ok`` is False when the staged target must be used."""

    def __init__(self, em: Emitter, stages: list | None = None):
        self.em = em
        self.stages = list(em.stages if stages is None else stages)
        self.phases: list[Phase] = []
        self.ok = True
        self.why = ""
        try:
            self._plan()
        except _NoFusion as e:
            self.ok, self.why = False, str(e)

    # -------------------------------------------------------------- analysis
    def _lambda_of(self, name_expr):
        em = self.em
        if not isinstance(name_expr, F.Name) or em.syms.get(name_expr.id, Sym("", "", None)).kind != "lambda":
            raise _NoFusion("map / reduce function is not a named lambda")
        return em.syms[name_expr.id]

    def _scalar_deps(self, node, seen=None) -> set:
        """Names of reduced symbols an expression (or lambda body) depends on."""
        em, out = self.em, set()
        seen = seen if seen is not None else set()
        for n in _walk(node):
            if isinstance(n, F.Name) and n.id in em.syms and n.id not in seen:
                s = em.syms[n.id]
                seen.add(n.id)
                if s.kind == "reduced":
                    out.add(n.id)
                elif s.kind == "derived":
                    out |= self._scalar_deps(s.expr, seen)
                elif s.kind == "lambda":
                    out |= self._scalar_deps(s.expr.body, seen)
                elif s.kind == "vector" and s.bits is not None:
                    out |= self._scalar_deps(s.bits, seen)
        return out

    def _vector_reads(self, lam: F.Lambda, own_index: str | None):
        """(vectors read at the own index, vectors read at any other index)."""
        em = self.em
        own, other = set(), set()
        for n in _walk(lam.body):
            if isinstance(n, F.Index) and isinstance(n.base, F.Name) and \
                    em.syms.get(n.base.id, Sym("", "", None)).kind in ("param_vector", "vector"):
                if own_index is not None and isinstance(n.idx, F.Name) and n.idx.id == own_index:
                    own.add(n.base.id)
                else:
                    other.add(n.base.id)
            elif isinstance(n, F.Call) and n.fn in em.syms and em.syms[n.fn].kind == "lambda":
                raise _NoFusion("a lambda that calls another lambda")
        return own, other

    def _count_of_map(self, m: F.Map) -> str:
        em = self.em
        if m.vec is not None:
            if not isinstance(m.vec, F.Name):
                raise _NoFusion("map over an expression")
            return f"c.n_{m.vec.id}"
        if isinstance(m.count, F.SizeOf) and isinstance(m.count.base, F.Name):
            return f"c.n_{m.count.base.id}"
        return f"(uint64_t)({em.expr(m.count, set())})"

    def _plan(self):
        em = self.em
        cur: Phase | None = None

        def close():
            nonlocal cur
            if cur is not None and cur.items:
                self.phases.append(cur)
            cur = None

        for st in self.stages:
            if st[0] in ("topk", "scatter"):
                raise _NoFusion("library-lowered stage")
            if st[0] == "reduce":
                for s in st[1]:
                    r: F.Reduce = s.expr
                    if not isinstance(r.vec, F.Name):
                        raise _NoFusion("reduce over an expression")
                    count = f"c.n_{r.vec.id}"
                    if cur is not None and r.vec.id in cur.written:
                        count = cur.count      # just produced over the phase's range
                    needs = self._scalar_deps(r.init)
                    if not (isinstance(r.fn, F.Name) and r.fn.id in ("smaller", "greater", "sum")
                            and r.fn.id not in em.syms):
                        lam = self._lambda_of(r.fn)
                        needs |= self._scalar_deps(lam.expr.body)
                        if self._vector_reads(lam.expr, None)[1]:
                            raise _NoFusion("a reducer that reads vectors")
                    if cur is None or cur.count != count or (needs & cur.reduced) or \
                            r.vec.id in cur.read_elsewhere:
                        close()
                        cur = Phase(count)
                    cur.items.append(Item("reduce", sym=s))
                    cur.reduced.add(s.name)
                continue
            target, m = em.maps[st[1]]
            lam = self._lambda_of(m.fn).expr
            count = self._count_of_map(m)
            if cur is not None and m.vec is not None and m.vec.id in cur.written:
                count = cur.count
            own_idx = lam.params[0][1] if (m.vec is None and lam.params) else None
            own, other = self._vector_reads(lam, own_idx)
            if m.vec is not None:
                own.add(m.vec.id)
            needs = self._scalar_deps(lam.body) | self._scalar_deps(em.syms[target].bits)
            if m.count is not None:
                needs |= self._scalar_deps(m.count)
            fresh = cur is None or cur.count != count or (needs & cur.reduced) or \
                bool(other & set(cur.written)) or target in cur.read_elsewhere or \
                (target in other)
            if fresh:
                close()
                cur = Phase(count)
            cur.items.append(Item("map", target=target, m=m, index=st[1]))
            cur.written.append(target)
            cur.read_elsewhere |= other
        close()
        if not self.phases:
            raise _NoFusion("nothing to launch")


class _NoFusion(Exception):
    pass


def fused_segments(em: Emitter) -> list:
    """For a function that keeps the staged target because of a library-lowered stage:
    the runs of consecutive ``map`` stages between the library calls that can still be
    one kernel.  Returns [(index of the run's first stage, number of stages, FusedPlan)].
    Kept simple on purpose: the function has no reduction, the run has at least two
    maps, none of them draws random numbers (the call sites are numbered per target)
    and the run plans as a single phase, so the kernel needs no grid barrier."""
    if em.reduces:
        return []
    out, i, n = [], 0, len(em.stages)
    while i < n:
        j = i
        while j < n and em.stages[j][0] == "map":
            j += 1
        run = em.stages[i:j]
        if len(run) >= 2:
            rnd = False
            for st in run:
                lam = em.syms.get(getattr(em.maps[st[1]][1].fn, "id", ""), None)
                if lam is None or any(isinstance(x, F.Random) for x in _walk(lam.expr.body)):
                    rnd = True
            plan = None if rnd else FusedPlan(em, run)
            if plan is not None and plan.ok and len(plan.phases) == 1:
                out.append((i, len(run), plan))
        i = max(j, i + 1)
    return out


class FusedGen:
    """Emits the fused kernel and its launch for a plan that is ``ok``."""

    def __init__(self, plan: FusedPlan, tag: str = "fused", write_header: bool = True):
        self.plan, self.em = plan, plan.em
        self.name = self.em.fn.name
        self.tag = tag                    # kernel name: <function>_<tag>_kernel
        self.write_header = write_header  # the launch that runs last writes the concat headers

    # ------------------------------------------------------------ helpers
    def _apply(self, r: F.Reduce, a: str, b: str) -> str:
        return self.em._apply(r.fn, a, b)

    def _prologue_lines(self):
        rows = self.em.prologue().replace("scalars[", "red[").splitlines()
        return [r for r in rows if r.strip() not in ("Ctx c;", "c.seed = seed;")]

    def _elem_type(self, vec: str) -> str:
        s = self.em.syms[vec]
        return "uint32_t" if s.bits is not None else C_TYPES[s.type.name]

    # ------------------------------------------------------------- phases
    def _phase(self, pi: int, ph: Phase, last: bool) -> str:
        em = self.em
        need_in: dict[str, None] = {}
        need_frag: dict[str, None] = {}
        sites: list[int] = []
        fwd: dict[str, str] = {}
        body = []
        last_writer = {it.target: k for k, it in enumerate(ph.items) if it.kind == "map"}

        def index_hook(sym, idx, local):
            own = em._own
            if own is None or not (isinstance(idx, F.Name) and idx.id == own and idx.id in local):
                return None
            if sym.name in fwd:
                return fwd[sym.name]
            if sym.bits is None:
                need_in[sym.name] = None
                return f"in_{sym.name}[u][e]"
            return frag_value(sym)

        def frag_value(sym):
            # a packed input read at the own index: the group's fragment is loaded once
            need_frag[sym.name] = None
            b = f"(uint32_t)({em.expr(sym.bits, set())})"
            return f"((fr_{sym.name}[u] >> (e * {b})) & ((1u << {b}) - 1u))"

        def random_hook(site):
            sites.append(site)
            return f"hipress::u01(rg{site}.v[e])"

        def stream_value(vec: str) -> str:
            if vec in fwd:
                return fwd[vec]
            s = em.syms[vec]
            if s.bits is None:
                need_in[vec] = None
                return f"in_{vec}[u][e]"
            return frag_value(s)

        em._index_hook, em._random_hook = index_hook, random_hook
        decls, stores = [], []
        try:
            for k, it in enumerate(ph.items):
                if it.kind == "reduce":
                    r: F.Reduce = it.sym.expr
                    ty = C_TYPES[it.sym.type.name]
                    body.append(f"        acc_{it.sym.name} = "
                                f"{self._apply(r, 'acc_' + it.sym.name, '(' + ty + ')' + stream_value(r.vec.id))};")
                    continue
                tgt = em.syms[it.target]
                lam_sym = em.syms[it.m.fn.id]
                lam: F.Lambda = lam_sym.expr
                sub = tgt.bits is not None
                rty = "uint32_t" if sub else C_TYPES[tgt.type.name]
                lret = "uint32_t" if lam.ret.is_subbyte() else C_TYPES[lam.ret.name]
                var = f"r{pi}_{k}"
                decls.append(f"      {rty} {var}[4] = {{0, 0, 0, 0}};")
                pty, pname = lam.params[0]
                local = {pname}
                if it.m.vec is not None:       # map over a vector: the parameter is the element
                    em._own = None
                    pinit = f"({C_TYPES[pty.name]})({stream_value(it.m.vec.id)})"
                else:
                    em._own = pname
                    pinit = f"({C_TYPES[pty.name]})i"
                em._counter = pname
                em._return_to = "res"
                code = em.stmts(lam.body, local, lam.ret.is_subbyte(), indent="            ")
                em._return_to = None
                mask = ""
                if sub:
                    mask = f" & ((1u << (uint32_t)({em.expr(tgt.bits, set())})) - 1u)"
                body.append(f"""        {{  // {it.target} = map(..., {lam_sym.name})
          const {C_TYPES[pty.name]} l_{pname} = {pinit};
          {lret} res = 0;
          do {{
{code}
          }} while (0);
          {var}[e] = (({rty})res){mask};
        }}""")
                fwd[it.target] = f"{var}[e]"
                if last_writer[it.target] == k:
                    if sub:
                        bits = f"(uint32_t)({em.expr(tgt.bits, set())})"
                        stores.append(f"""      {{
        const uint32_t bits = {bits};
        const uint32_t frag = {var}[0] | ({var}[1] << bits) | ({var}[2] << (2 * bits)) | ({var}[3] << (3 * bits));
        compll_pack_store(c.v_{it.target}, (count * bits + 7) / 8, q, frag, bits);
      }}""")
                    else:
                        stores.append(f"      compll_store4(c.v_{it.target}, i0, count, {var});")
        finally:
            em._index_hook = em._random_hook = None
            em._own = None
            em._return_to = None
        # U groups of four elements per thread and trip, every load of a trip issued before
        # the first result is computed (a map only reads its own elements of the vectors
        # it also writes, so hoisting the loads over the stores is safe).  Measured at
        # 256 MB: a phase whose only inputs are packed fragments (the decodes, bound by
        # their stores) gains from four groups in flight (TbqDecode 0.075 -> 0.061 ms,
        # OnebitDecode 0.069 -> 0.057 ms); a phase that also streams a float vector in
        # (decode-accumulate, the encoders) lost up to 25 % and keeps one.
        U = 4 if not need_in else 1
        larr = [f"      {C_TYPES[em.syms[v].type.name]} in_{v}[{U}][4];" for v in need_in] + \
               [f"      uint32_t fr_{v}[{U}];" for v in need_frag]
        loads = [f"        compll_load4(c.v_{v}, i0, count, in_{v}[u]);" for v in need_in]
        for v in need_frag:
            b = f"(uint32_t)({em.expr(em.syms[v].bits, set())})"
            loads.append(f"        fr_{v}[u] = compll_load_frag(c.v_{v}, (c.n_{v} * {b} + 7) / 8, q, {b});")
        rngs = [f"      const hipress::Philox4 rg{s} = compll_rand4(c.seed, q, {s}u);" for s in sorted(set(sites))]
        reds = [it.sym for it in ph.items if it.kind == "reduce"]
        acc_init = [f"    {C_TYPES[s.type.name]} acc_{s.name} = ({C_TYPES[s.type.name]})"
                    f"({em.expr(s.expr.init, set())});" for s in reds]
        nl = "\n"
        header = ""
        if last and self.write_header:
            rows = []
            for tname, fields, _ in em.concats:
                for fname, off in fields:
                    s = em.syms[fname]
                    rows.append(f"      compll_store<{C_TYPES[s.type.name]}>(reinterpret_cast<uint8_t*>"
                                f"(p_{tname}) + {off}, c.v_{fname});")
            if rows:
                header = "    if (blockIdx.x == 0 && threadIdx.x == 0) {\n" + nl.join(rows) + "\n    }\n"
        out = f"""  {{  // ---- phase {pi}: {', '.join((it.target if it.kind == 'map' else 'reduce ' + it.sym.name) for it in ph.items)}
{header}    const uint64_t count = {ph.count};
    const uint64_t groups = (count + 3) / 4;
{nl.join(acc_init)}
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t qb0 = (uint64_t)blockIdx.x * blockDim.x; qb0 < groups; qb0 += stride * {U}) {{
{nl.join(larr)}
#pragma unroll
      for (int u = 0; u < {U}; ++u) {{   // past the end the loads return zeros and touch nothing
        const uint64_t q = qb0 + u * stride + threadIdx.x;
        const uint64_t i0 = q * 4;
        (void)q; (void)i0;
{nl.join(loads)}
      }}
#pragma unroll
      for (int u = 0; u < {U}; ++u) {{
      const uint64_t qb = qb0 + u * stride;   // the same for the whole block
      if (qb >= groups) break;
      const uint64_t q = qb + threadIdx.x;
      const uint64_t i0 = q * 4;
{nl.join(rngs)}
{nl.join(decls)}
#pragma unroll
      for (int e = 0; e < 4; ++e) {{
        const uint64_t i = i0 + e;
        if (i >= count) continue;
{nl.join(body)}
      }}
{nl.join(stores)}
      }}
    }}
{self._block_reduce(reds)}  }}
"""
        return out

    def _block_reduce(self, reds) -> str:
        if not reds:
            return ""
        rows = ["    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;",
                "    for (int off = 16; off > 0; off >>= 1) {"]
        for s in reds:
            ty = C_TYPES[s.type.name]
            rows.append(f"      {{ {ty} o = __shfl_xor_sync(0xffffffffu, acc_{s.name}, off); "
                        f"acc_{s.name} = {self._apply(s.expr, 'acc_' + s.name, 'o')}; }}")
        rows.append("    }")
        rows.append("    __syncthreads();")
        rows.append("    if (lane == 0) { " + " ".join(f"sh[{s.slot}][warp] = (float)acc_{s.name};" for s in reds) + " }")
        rows.append("    __syncthreads();")
        rows.append("    if (threadIdx.x == 0) {")
        for s in reds:
            ty = C_TYPES[s.type.name]
            rows.append(f"      {{ {ty} a = ({ty})sh[{s.slot}][0]; for (int w = 1; w < 8; ++w) "
                        f"a = {self._apply(s.expr, 'a', '(' + ty + ')sh[' + str(s.slot) + '][w]')}; "
                        f"partials[{s.slot} * gridDim.x + blockIdx.x] = (float)a; }}")
        rows.append("    }")
        return "\n".join(rows) + "\n"

    def _fold(self, reds) -> str:
        """Behind the barrier: every block folds the per-block partials itself."""
        rows = []
        for s in reds:
            ty = C_TYPES[s.type.name]
            init = self.em.expr(s.expr.init, set())
            rows.append(f"""  {{
    {ty} a = ({ty})({init});
    if (threadIdx.x < 32) {{
      for (unsigned w = threadIdx.x; w < gridDim.x; w += 32)
        a = {self._apply(s.expr, 'a', '(' + ty + ')__ldcg(&partials[' + str(s.slot) + ' * gridDim.x + w])')};
      for (int off = 16; off > 0; off >>= 1) {{
        {ty} o = __shfl_xor_sync(0xffffffffu, a, off);
        a = {self._apply(s.expr, 'a', 'o')};
      }}
      if (threadIdx.x == 0) sh[{s.slot}][0] = (float)a;
    }}
    __syncthreads();
    red[{s.slot}] = sh[{s.slot}][0];
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0) scalars[{s.slot}] = red[{s.slot}];
  }}""")
        return "\n".join(rows)

    # -------------------------------------------------------------- kernel
    def kernel_source(self) -> str:
        em, name = self.em, self.name
        phases = self.plan.phases
        nred = max(len(em.reduces), 1)
        pro = "\n".join(self._prologue_lines())
        parts = []
        for pi, ph in enumerate(phases):
            parts.append(self._phase(pi, ph, pi == len(phases) - 1))
            if pi != len(phases) - 1:
                reds = [it.sym for it in ph.items if it.kind == "reduce"]
                parts.append(f"  compll_grid_sync(sync, gen, sync + 2);\n{self._fold(reds)}\n{pro}\n")
        tail = ""
        if len(phases) > 1:
            tail = """  // the last block to leave clears the barrier words for the next launch
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(sync + 1, 1u) == gridDim.x - 1) {
    sync[0] = 0;
    sync[1] = 0;
  }
"""
        return f"""
// One launch for the whole function: {len(phases)} phase(s){', grid barriers in between' if len(phases) > 1 else ''}.
__global__ void __launch_bounds__(256) {name}_{self.tag}_kernel({em.kernel_params()}, float* partials,
                                                       unsigned int* sync) {{
  __shared__ float sh[{nred}][8];
  float red[{nred}];
  for (int k = 0; k < {nred}; ++k) red[k] = 0.0f;
  unsigned int gen = 0;
  (void)gen; (void)sh; (void)partials; (void)sync;
  Ctx c;
  c.seed = seed;
{pro}
{''.join(parts)}{tail}}}
"""

    def launch_rows(self) -> str:
        """Body of the launcher: grid sizing and the (cooperative) launch."""
        name = self.name
        coop = len(self.plan.phases) > 1
        most_rows = "\n".join(f"    if (n_{pname} > most) most = n_{pname};"
                              for ty, pname in self.em.fn.params if ty.vector)
        return f"""  {{
    static int cap[64] = {{0}};           // blocks the device holds at once
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cap[dev] == 0) {{
      int sms = 0, per = 0;
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, compll_gen_{name}::{name}_{self.tag}_kernel, 256, 0);
      cap[dev] = per * sms > 0 ? per * sms : 1;
    }}
    uint64_t most = work;
{most_rows}
    int fgrid = (int)((most / 4 + 255) / 256);
    if (fgrid < 1) fgrid = 1;
    if (fgrid > cap[dev]) fgrid = cap[dev];
    if (fgrid > kMaxBlocks) fgrid = kMaxBlocks;
    unsigned int* sync = ticket;
    void* args[] = {{{', '.join('(void*)&' + a for a in self._arg_names())}, (void*)&partials, (void*)&sync}};
    cudaError_t e = {'cudaLaunchCooperativeKernel' if coop else 'cudaLaunchKernel'}(
        (const void*)compll_gen_{name}::{name}_{self.tag}_kernel, dim3(fgrid), dim3(256), args, 0, st);
    if (e != cudaSuccess) return (int)e;
  }}"""

    def _arg_names(self):
        a = []
        for ty, pname in self.em.fn.params:
            a += [f"p_{pname}", f"n_{pname}"] if ty.vector else [f"p_{pname}"]
        return a + ["scalars", "seed"]
