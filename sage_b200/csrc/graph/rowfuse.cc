// Whole-row programs: analysis of the graph, CUDA C generation, launch.  See rowfuse.h.
//
// Value classes over the common row space (R rows of C contiguous elements; a tensor of any rank whose
// last axis has C elements and whose leading axes multiply to R is such a space, e.g. [32, 128, 768]):
//   Full    R * C elements, last extent C     C values per row, spread over the block's threads in registers
//   Row     R elements ([.., 1] or [..])      one value per row, held by every thread
//   Scalar  one element                       one value, held by every thread
// Operators accepted (anything else makes the graph ineligible and the evaluator compiles it the
// ordinary way): maps (src/ops/map.rs) whose operands are of the output's class or broadcast into it;
// reshape / expand / squeeze / unsqueeze that keep a value per-row or per-graph (src/ops/core.rs:203-476;
// they generate no code); reductions over axis 1 (src/ops/reduce.rs:258-325) with the reference's
// accumulator rule; gather and scatter along axis 1 with one index per row (src/ops/core.rs:613-834).
#include "rowfuse.h"

#include <cstdio>
#include <cstdlib>
#include <sstream>

namespace sage {

const char *map_prelude_text();
int view_op_kind(const Operator &op);
int index_op_axis(const Operator &op, bool scatter);
bool reduce_op_info(const Operator &op, int *kind, std::vector<int> *axes);

namespace {

enum Cls { Scalar = 0, Row = 1, Full = 2 };
enum Kind { KLeaf, KAlias, KMap, KReduce, KGather, KScatter };

struct Val {
    Kind kind = KLeaf;
    Cls cls = Scalar;
    int dtype = SAGE_F32;
    Var var;
    std::vector<int> args;
    std::string expr;  // KMap: C expression over x0..xn
    int red = 0;       // KReduce: ops::Red
    int input = -1, output = -1;
    bool bcast_leaf = false;  // KLeaf: a Full-shaped view with last stride 0, read as a value per row
};

const char *ctype(int dt) { return dt == SAGE_F32 ? "float" : dt == SAGE_I32 ? "int" : "uint"; }
const char *vtype(int dt) { return dt == SAGE_F32 ? "float4" : dt == SAGE_I32 ? "int4" : "uint4"; }

bool classify(const Array &e, long long R, long long C, Cls *c) {
    long long size = 1;
    for (long long x : e) size *= x;
    if (size == 1) *c = Scalar;
    else if (size == R * C && e.back() == C) *c = Full;
    else if (size == R) *c = Row;  // R != R * C and a Full value has more elements, so the three cases are disjoint
    else return false;
    return true;
}

constexpr size_t kMaxValues = 256;

}  // namespace

struct RowProgram {
    long long rows = 0, cols = 0;
    int threads = 0, nv = 0, vec = 0;
    std::vector<Val> vals;  // topological order
    std::vector<int> in_val, out_val;
    int n_map = 0, n_reduce = 0, n_index = 0;
    std::string source;
    uint32_t stage_bytes = 0;  // dynamic shared memory of the prefetch stages (0: inputs are loaded directly)
    Module *module = nullptr;
    Context *owner = nullptr;
    int resident = 1;  // blocks per SM

    int resolve(int id) const {
        while (vals[id].kind == KAlias) id = vals[id].args[0];
        return id;
    }
    std::string ref(int id) const {
        id = resolve(id);
        return "v" + std::to_string(id) + (vals[id].cls == Full ? "[e]" : "");
    }
};

namespace {

struct Builder {
    RowProgram &p;
    std::unordered_set<Origin *> evaluated;
    std::unordered_map<Origin *, int> memo;
    bool ok = true;

    int fail() {
        ok = false;
        return -1;
    }

    int add(const Var &v) {
        if (!ok) return -1;
        auto it = memo.find(v.key());
        if (it != memo.end()) return it->second;
        if (p.vals.size() >= kMaxValues) return fail();
        Val val;
        val.var = v;
        val.dtype = v.dtype();
        if (!classify(v.extents(), p.rows, p.cols, &val.cls)) return fail();
        if (v.is_data() || evaluated.count(v.key())) {
            val.kind = KLeaf;
            val.input = (int)p.in_val.size();
            // A materialised view that repeats one value along the row (expand of a [.., 1] tensor: the state
            // keeps the source's buffer, last stride 0): read as one value per row, never copied out.
            const Shape &sh = v.desc.shape;
            if (val.cls == Full && sh.strides.back() == 0) {
                Array lead(sh.extents.begin(), sh.extents.end() - 1);
                const Array dflt = Shape::default_strides(lead);
                bool rows_contiguous = true;
                for (size_t i = 0; i < lead.size(); ++i)
                    if (lead[i] > 1 && sh.strides[i] != dflt[i]) rows_contiguous = false;
                if (!rows_contiguous) return fail();
                val.cls = Row;
                val.bcast_leaf = true;
            }
        } else {
            const Operator &op = *v.origin->op;
            const std::vector<Var> &in = v.origin->inputs;
            for (const Var &a : in) {
                const int id = add(a);
                if (!ok) return -1;
                val.args.push_back(id);
            }
            auto cls_of = [&](int i) { return p.vals[p.resolve(val.args[i])].cls; };
            int red_kind, vk;
            std::vector<int> axes;
            if (const MapExpr *e = map_expr_of(op)) {
                for (size_t i = 0; i < in.size(); ++i)
                    if (cls_of((int)i) > val.cls) return fail();
                val.kind = KMap;
                val.expr = map_expr_text(*e);
                ++p.n_map;
            } else if ((vk = view_op_kind(op)) >= 0) {
                if (vk == 2 || vk == 5) return fail();  // permute, slice
                const Array &ie = in[0].extents();
                if (vk == 1) {
                    // expand: from one element, or from a value per row laid out with a trailing unit axis
                    // (a vector along the row axis, e.g. a bias [C], has R == C elements at most by accident)
                    if (!(in[0].size() == 1 || (in[0].size() == p.rows && ie.back() == 1))) return fail();
                } else if (p.vals[val.args[0]].cls != val.cls) {
                    return fail();  // reshape / squeeze / unsqueeze keep a value in its class (rows stay rows)
                }
                val.kind = KAlias;
                val.cls = cls_of(0);
            } else if (reduce_op_info(op, &red_kind, &axes)) {
                const Array &ie = in[0].extents();
                if (v.dtype() != SAGE_F32 || axes.size() != 1 || axes[0] != in[0].rank() - 1 || val.cls != Row) return fail();
                // over the row axis of a Full value (which really has those extents: not a broadcast standing
                // for them), or over the trailing unit axis of a value per row
                if (in[0].size() == p.rows * p.cols ? (ie.back() != p.cols || cls_of(0) != Full) : (in[0].size() != p.rows || ie.back() != 1))
                    return fail();
                val.kind = KReduce;
                val.red = red_kind;
                ++p.n_reduce;
            } else if (index_op_axis(op, false) == in[0].rank() - 1 && index_op_axis(op, false) >= 0) {
                const Array &ie = in[1].extents();
                if (in[0].size() != p.rows * p.cols || in[0].extents().back() != p.cols || cls_of(0) != Full || in[1].size() != p.rows || ie.back() != 1)
                    return fail();
                val.kind = KGather;
                ++p.n_index;
            } else if (index_op_axis(op, true) == in[0].rank() - 1 && index_op_axis(op, true) >= 0) {
                const Array &ie = in[1].extents();
                if (val.cls != Full || v.dtype() != SAGE_F32 || in[1].size() != p.rows || ie.back() != 1 || cls_of(0) == Full) return fail();
                val.kind = KScatter;
                ++p.n_index;
            } else {
                return fail();
            }
        }
        const int id = (int)p.vals.size();
        if (val.kind == KLeaf) p.in_val.push_back(id);
        p.vals.push_back(val);
        memo[v.key()] = id;
        return id;
    }
};

// Cheap screen before any allocation: every operator below the targets is of an accepted family, and
// the graph is small.  Also finds the row space: the largest value is a Full one, its last extent is C.
bool screen(const std::vector<Var> &targets, const std::unordered_set<Origin *> &evaluated, bool maps_suffice, long long *R, long long *C) {
    std::unordered_set<Origin *> seen;
    std::vector<Var> stack = targets;
    bool reduces = false;
    long long largest = 0;
    while (!stack.empty()) {
        Var v = stack.back();
        stack.pop_back();
        if (!seen.insert(v.key()).second) continue;
        if (seen.size() > kMaxValues) return false;
        if (v.size() > largest && v.rank() >= 1) {
            largest = v.size();
            *C = v.extents().back();
            *R = largest / *C;
        }
        if (v.is_data() || evaluated.count(v.key())) continue;
        const Operator &op = *v.origin->op;
        int kind;
        std::vector<int> axes;
        if (reduce_op_info(op, &kind, &axes)) reduces = true;
        else if (index_op_axis(op, false) >= 0 || index_op_axis(op, true) >= 0) reduces = true;
        else if (!map_expr_of(op) && view_op_kind(op) < 0) return false;
        for (const Var &a : v.origin->inputs) stack.push_back(a);
    }
    return largest > 0 && *R > 1 && *C > 1 && (reduces || maps_suffice);
}

void emit(RowProgram &p) {
    std::ostringstream s;
    const int E = p.nv * p.vec;
    s << map_prelude_text();
    s << "#define RP_C " << p.cols << "\n#define RP_T " << p.threads << "\n#define RP_NV " << p.nv << "\n#define RP_VEC " << p.vec << "\n";
    s << "#define RP_E " << E << "\n";
    int wp2 = 1;
    while (wp2 < p.threads / 32) wp2 *= 2;
    s << "#define RP_WP2 " << wp2 << "\n";
    s << "#define RP_WHOLE " << ((long long)E * p.threads == p.cols ? 1 : 0) << "\n";
    s << "#define RP_COL(e) ((((e) / RP_VEC) * RP_T + (int)threadIdx.x) * RP_VEC + (e) % RP_VEC)\n";
    s << "#define RP_OK(e) (RP_WHOLE || RP_COL(e) < RP_C)\n";
    s << "struct RowP { long long rows; int compat; int pad; const void *in[" << std::max<size_t>(1, p.in_val.size()) << "]; void *out["
      << std::max<size_t>(1, p.out_val.size()) << "]; float *out_hi[" << std::max<size_t>(1, p.out_val.size()) << "]; long long out_plane["
      << std::max<size_t>(1, p.out_val.size()) << "]; };\n";
    s << R"(template <int K> SG float rp_apply(float a, float b) { return K == 0 ? a + b : K == 1 ? a * b : K == 2 ? fmaxf(a, b) : fminf(a, b); }
template <int K> SG float rp_identity() { return K == 0 ? 0.f : K == 1 ? 1.f : K == 2 ? __int_as_float(0xff800000) : __int_as_float(0x7f800000); }
// Every thread returns the same value: a butterfly combines the same pairs in every lane, and every
// group of RP_WP2 lanes (RP_WP2 = warps per block rounded up to a power of two) holds all the warp
// partials and runs the same second butterfly over them.
template <int K> SG float rp_reduce(float acc, float *sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc = rp_apply<K>(acc, __shfl_xor_sync(0xffffffffu, acc, o));
  if (RP_T > 32) {
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    const int w = threadIdx.x & (RP_WP2 - 1);
    acc = w < RP_T / 32 ? sh[w] : rp_identity<K>();
#pragma unroll
    for (int o = RP_WP2 / 2; o > 0; o >>= 1) acc = rp_apply<K>(acc, __shfl_xor_sync(0xffffffffu, acc, o));
  }
  return acc;
}
// One barrier per exchange: every exchange of the program owns a scratch slot per row parity, so a slot
// is rewritten two rows later, and the barrier of the row in between orders that write after every
// thread's reads.
SG void rp_copy16(void *smem, const void *gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
SG uint rp_bits(float x) { return __float_as_uint(x); }
SG uint rp_bits(int x) { return (uint)x; }
SG uint rp_bits(uint x) { return x; }
SG void rp_from(uint b, float *x) { *x = __uint_as_float(b); }
SG void rp_from(uint b, int *x) { *x = (int)b; }
SG void rp_from(uint b, uint *x) { *x = b; }
SG void rp_prefetch(const RowP &p, long long row, uint4 *stage);
)";
    // exchanges (block reductions, gathers) get a scratch slot each; Full leaves a place in the prefetch stage
    std::vector<int> slot(p.vals.size(), -1), stage_of(p.vals.size(), -1);
    int n_red = 0, n_pick = 0, n_stage = 0;
    for (size_t id = 0; id < p.vals.size(); ++id) {
        const Val &v = p.vals[id];
        if (v.kind == KReduce && p.vals[p.resolve(v.args[0])].cls == Full) slot[id] = n_red++;
        if (v.kind == KGather) slot[id] = n_pick++;
        if (v.kind == KLeaf && v.cls == Full) stage_of[id] = n_stage++;
    }
    // Prefetch: while a row is being computed, the next row of every Full input is already on its way
    // into shared memory (cp.async, 16 bytes per thread and vector; each thread later reads back exactly
    // what it copied, so no barrier is involved).  Two stages alternate by row parity.
    p.stage_bytes = 0;
    if (p.vec == 4 && n_stage > 0) {
        const size_t bytes = (size_t)2 * n_stage * p.nv * p.threads * 16;
        if (bytes <= 96 * 1024) p.stage_bytes = (uint32_t)bytes;
    }
    s << "#define RP_STAGE " << (size_t)n_stage * p.nv * p.threads << "\n";
    // at least as many blocks per SM as ~80 registers per thread allow: more warps to hide the latency of
    // exp, shared memory and shuffles (the kernels run at low occupancy by construction)
    s << "extern \"C\" __global__ void __launch_bounds__(RP_T, " << std::max(1, 65536 / (p.threads * 80)) << ") sage_row_program(const RowP p) {\n"
      << "  asm volatile(\"griddepcontrol.launch_dependents;\" ::: \"memory\");\n"
      << "  asm volatile(\"griddepcontrol.wait;\" ::: \"memory\");\n"
      << "  __shared__ float sh[2][" << std::max(1, n_red) << "][32];\n  __shared__ uint sh_pick[2][" << std::max(1, n_pick) << "];\n";
    if (p.stage_bytes)
        s << "  extern __shared__ uint4 rp_stage[];\n  if ((long long)blockIdx.x < p.rows) rp_prefetch(p, blockIdx.x, rp_stage);\n";
    s << "  int par = 0;\n  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x, par ^= 1) {\n";
    if (p.stage_bytes)
        s << "    asm volatile(\"cp.async.wait_group 0;\" ::: \"memory\");\n    const uint4 *cur = rp_stage + par * RP_STAGE;\n"
          << "    if (row + gridDim.x < p.rows) rp_prefetch(p, row + gridDim.x, rp_stage + (par ^ 1) * RP_STAGE);\n";
    const char *comp[4] = {"x", "y", "z", "w"};
    for (size_t id = 0; id < p.vals.size(); ++id) {
        const Val &v = p.vals[id];
        const char *T = ctype(v.dtype);
        const std::string name = "v" + std::to_string(id);
        switch (v.kind) {
        case KAlias: break;
        case KLeaf:
            if (v.cls == Full) {
                if (p.stage_bytes) {
                    s << "    " << T << " " << name << "[RP_E];\n#pragma unroll\n    for (int j = 0; j < RP_NV; ++j) {\n"
                      << "      const int c0 = (j * RP_T + (int)threadIdx.x) * 4;\n      uint4 t = {0u, 0u, 0u, 0u};\n"
                      << "      if (RP_WHOLE || c0 < RP_C) t = cur[(" << stage_of[id] << " * RP_NV + j) * RP_T + threadIdx.x];\n";
                    for (int q = 0; q < 4; ++q) s << "      rp_from(t." << comp[q] << ", &" << name << "[4 * j + " << q << "]);\n";
                    s << "    }\n";
                    break;
                }
                s << "    " << T << " " << name << "[RP_E];\n    {\n      const " << T << " *src = (const " << T << " *)p.in[" << v.input
                  << "] + row * RP_C;\n#pragma unroll\n      for (int j = 0; j < RP_NV; ++j) {\n"
                  << "        const int c0 = (j * RP_T + (int)threadIdx.x) * RP_VEC;\n";
                if (p.vec == 4) {
                    s << "        " << vtype(v.dtype) << " t = {0, 0, 0, 0};\n        if (RP_WHOLE || c0 < RP_C) t = __ldg(reinterpret_cast<const "
                      << vtype(v.dtype) << " *>(src + c0));\n";
                    for (int q = 0; q < 4; ++q) s << "        " << name << "[4 * j + " << q << "] = t." << comp[q] << ";\n";
                } else {
                    s << "        " << name << "[j] = (RP_WHOLE || c0 < RP_C) ? __ldg(src + c0) : (" << T << ")0;\n";
                }
                s << "      }\n    }\n";
            } else {
                s << "    const " << T << " " << name << " = __ldg((const " << T << " *)p.in[" << v.input << "]" << (v.cls == Row ? " + row" : "")
                  << ");\n";
            }
            break;
        case KMap: {
            std::ostringstream body;
            for (size_t i = 0; i < v.args.size(); ++i)
                body << "const " << ctype(p.vals[p.resolve(v.args[i])].dtype) << " x" << i << " = " << p.ref(v.args[i]) << "; ";
            if (v.cls == Full)
                s << "    " << T << " " << name << "[RP_E];\n#pragma unroll\n    for (int e = 0; e < RP_E; ++e) { " << body.str() << name << "[e] = ("
                  << T << ")(" << v.expr << "); }\n";
            else
                s << "    " << T << " " << name << ";\n    { " << body.str() << name << " = (" << T << ")(" << v.expr << "); }\n";
            break;
        }
        case KReduce: {
            const int a = p.resolve(v.args[0]);
            s << "    float " << name << ";\n    {\n";
            if (p.vals[a].cls == Full) {
                s << "      float acc = rp_identity<" << v.red << ">();\n#pragma unroll\n      for (int e = 0; e < RP_E; ++e) if (RP_OK(e)) acc = rp_apply<"
                  << v.red << ">(acc, v" << a << "[e]);\n      acc = rp_reduce<" << v.red << ">(acc, sh[par][" << slot[id] << "]);\n";
            } else {
                s << "      float acc = v" << a << ";\n";
            }
            // the reference's accumulator starts at 0 whatever the operation (src/ops/reduce.rs:292)
            s << "      " << name << " = p.compat ? rp_apply<" << v.red << ">(0.f, acc) : acc;\n    }\n";
            break;
        }
        case KGather: {
            const int a = p.resolve(v.args[0]);
            // an index outside the row picks nothing: the value is then whatever the slot held (the reference
            // reads out of bounds there)
            s << "    " << T << " " << name << ";\n    {\n      const uint pick = (uint)" << p.ref(v.args[1]) << ";\n#pragma unroll\n"
              << "      for (int e = 0; e < RP_E; ++e) if (RP_OK(e) && (uint)RP_COL(e) == pick) sh_pick[par][" << slot[id] << "] = rp_bits(v" << a
              << "[e]);\n      __syncthreads();\n      rp_from(sh_pick[par][" << slot[id] << "], &" << name << ");\n    }\n";
            break;
        }
        case KScatter:
            // into zeros, one index per row: 0 + x at the index (scatter adds, src/ops/core.rs:764-833), 0 elsewhere
            s << "    float " << name << "[RP_E];\n    {\n      const uint pick = (uint)" << p.ref(v.args[1]) << ";\n      const float put = 0.f + "
              << p.ref(v.args[0]) << ";\n#pragma unroll\n      for (int e = 0; e < RP_E; ++e) " << name
              << "[e] = (uint)RP_COL(e) == pick ? put : 0.f;\n    }\n";
            break;
        }
        if (v.output >= 0) {
            if (v.cls == Full) {
                s << "    {\n      " << T << " *dst = (" << T << " *)p.out[" << v.output << "] + row * RP_C;\n#pragma unroll\n"
                  << "      for (int j = 0; j < RP_NV; ++j) {\n        const int c0 = (j * RP_T + (int)threadIdx.x) * RP_VEC;\n"
                  << "        if (RP_WHOLE || c0 < RP_C) ";
                if (p.vec == 4) {
                    s << "{ " << vtype(v.dtype) << " t; ";
                    for (int q = 0; q < 4; ++q) s << "t." << comp[q] << " = " << name << "[4 * j + " << q << "]; ";
                    s << "*reinterpret_cast<" << vtype(v.dtype) << " *>(dst + c0) = t; }\n";
                } else {
                    s << "dst[c0] = " << name << "[j];\n";
                }
                s << "      }\n    }\n";
                if (v.dtype == SAGE_F32) {  // the tf32 planes of this output, when a tensor-core GEMM reads it next
                    s << "    if (p.out_hi[" << v.output << "]) {\n      float *hi = p.out_hi[" << v.output << "] + row * RP_C, *lo = hi + p.out_plane["
                      << v.output << "];\n#pragma unroll\n      for (int j = 0; j < RP_NV; ++j) {\n"
                      << "        const int c0 = (j * RP_T + (int)threadIdx.x) * RP_VEC;\n        if (RP_WHOLE || c0 < RP_C) {\n";
                    if (p.vec == 4) {
                        s << "          float4 h, l;\n";
                        for (int q = 0; q < 4; ++q)
                            s << "          sg_split_tf32(" << name << "[4 * j + " << q << "], &h." << comp[q] << ", &l." << comp[q] << ");\n";
                        s << "          *reinterpret_cast<float4 *>(hi + c0) = h;\n          *reinterpret_cast<float4 *>(lo + c0) = l;\n";
                    } else {
                        s << "          float h, l;\n          sg_split_tf32(" << name << "[j], &h, &l);\n          hi[c0] = h;\n          lo[c0] = l;\n";
                    }
                    s << "        }\n      }\n    }\n";
                }
            } else {
                s << "    if (threadIdx.x == 0) ((" << T << " *)p.out[" << v.output << "])[row] = " << name << ";\n";
            }
        }
    }
    s << "  }\n}\n";
    s << "SG void rp_prefetch(const RowP &p, long long row, uint4 *stage) {\n#pragma unroll\n  for (int j = 0; j < RP_NV; ++j) {\n"
      << "    const int c0 = (j * RP_T + (int)threadIdx.x) * 4;\n    if (RP_WHOLE || c0 < RP_C) {\n";
    for (size_t id = 0; id < p.vals.size(); ++id)
        if (stage_of[id] >= 0)
            s << "      rp_copy16(stage + (" << stage_of[id] << " * RP_NV + j) * RP_T + threadIdx.x, (const char *)p.in[" << p.vals[id].input
              << "] + (row * RP_C + c0) * 4);\n";
    s << "    }\n  }\n  asm volatile(\"cp.async.commit_group;\" ::: \"memory\");\n}\n";
    p.source = s.str();
}

}  // namespace

std::shared_ptr<RowProgram> row_program_build(const std::vector<Var> &evaluated, const std::vector<Var> &targets, bool whole_program, bool emit_source) {
    std::unordered_set<Origin *> ev;
    for (const Var &v : evaluated) ev.insert(v.key());
    long long R = 0, C = 0;
    if (!screen(targets, ev, !whole_program, &R, &C)) return nullptr;
    if (C < 32 || C > 16384) return nullptr;
    auto p = std::make_shared<RowProgram>();
    p->rows = R;
    p->cols = C;
    Builder b{*p, ev, {}, true};
    for (const Var &t : targets) {
        const int id = b.add(t);
        if (!b.ok) return nullptr;
        Val &v = p->vals[id];
        if (v.kind == KLeaf || v.kind == KAlias || v.cls == Scalar || v.output >= 0) return nullptr;
        v.output = (int)p->out_val.size();
        p->out_val.push_back(id);
    }
    bool full_leaf = false;
    for (int id : p->in_val) full_leaf = full_leaf || p->vals[id].cls == Full;
    if (whole_program && (!full_leaf || p->n_reduce + p->n_index == 0)) return nullptr;
    // Distribution of a row over the block: 128-bit accesses when the rows allow.  Elements per thread:
    // a block reduction costs every thread ~20 instructions whatever it holds, so few threads with
    // many elements keep the instruction count per element low (these kernels are as close to the
    // issue limit as to the HBM one); 16 per thread from 2048 columns, 8 from 1024, else 4.
    p->vec = C % 4 == 0 ? 4 : 1;
    const long long units = (C + p->vec - 1) / p->vec;  // vectors per row
    int elems = C >= 2048 ? 16 : C >= 1024 ? 8 : 4;
    if (const char *e = getenv("SAGE_ROW_PROGRAM_ELEMS")) elems = std::max(4, atoi(e));  // tuning aid
    p->nv = std::max(1, elems / p->vec);
    long long t = (units + p->nv - 1) / p->nv;
    while (t > 1024) {
        ++p->nv;
        t = (units + p->nv - 1) / p->nv;
    }
    if (p->nv * p->vec > 32) return nullptr;
    p->threads = (int)((t + 31) / 32 * 32);
    if (!emit_source) return p;  // analysis only: is the graph a row program, and over which space
    emit(*p);
    if (const char *path = getenv("SAGE_ROW_PROGRAM_DUMP")) {  // diagnostics: the generated source
        if (FILE *f = fopen(path, "w")) {
            fputs(p->source.c_str(), f);
            fclose(f);
        }
    }
    return p;
}

const std::string &row_program_source(const RowProgram &p) { return p.source; }

bool row_program_ready(const RowProgram &p, const Session &s) {
    for (int id : p.in_val)
        if (!p.vals[id].var.is_data() && !s.data.count(p.vals[id].var.key())) return false;
    return true;
}

std::string row_program_describe(const RowProgram &p) {
    std::ostringstream s;
    s << "row_program[" << p.rows << "x" << p.cols << "; " << p.threads << " threads x " << p.nv * p.vec << "]{" << p.n_map << " maps, " << p.n_reduce
      << " reductions, " << p.n_index << " gather/scatter}(" << p.in_val.size() << " inputs -> " << p.out_val.size() << " outputs)\n";
    return s.str();
}

void row_program_space(const RowProgram &p, long long *rows, long long *cols) {
    *rows = p.rows;
    *cols = p.cols;
}

int row_program_exchanges(const RowProgram &p) { return p.n_reduce + p.n_index; }

std::vector<Var> row_program_inputs(const RowProgram &p) {
    std::vector<Var> v;
    for (int id : p.in_val) v.push_back(p.vals[id].var);
    return v;
}

sage_status row_program_exec(RowProgram &p, Context &ctx, Session &s) {
    std::vector<Tensor> outs;
    sage_status st = row_program_run(p, ctx, [&](const Var &v, Tensor *t) { return s.get(v, t); }, &outs);
    if (st) return st;
    for (size_t i = 0; i < p.out_val.size(); ++i) {
        const Var &v = p.vals[p.out_val[i]].var;
        s.data[v.key()] = std::make_pair(v, outs[i]);
    }
    return SAGE_OK;
}

sage_status storage_planes_attach(Context &ctx, Storage &st);  // ops_gemm.cc

sage_status row_program_run(RowProgram &p, Context &ctx, const std::function<bool(const Var &, Tensor *)> &fetch, std::vector<Tensor> *outs_,
                            const std::vector<char> *planes) {
    if (p.source.empty()) return ctx.fail(SAGE_ERR_INVALID, "internal: row program was built for analysis only");
    if (p.owner != &ctx) {
        sage_status st = ctx.module_get(p.source, &p.module);
        if (st) return st;
        p.owner = &ctx;
        p.resident = ctx.blocks_per_sm(p.module, "sage_row_program", p.threads, p.stage_bytes);
    }
    std::vector<Tensor> keep;
    const size_t nin = std::max<size_t>(1, p.in_val.size()), nout = std::max<size_t>(1, p.out_val.size());
    std::vector<uint64_t> pb(2 + nin + 3 * nout, 0);  // rows, compat, in[], out[], out_hi[], out_plane[]
    pb[0] = (uint64_t)p.rows;
    pb[1] = (uint64_t)(ctx.opts().ref_compat ? 1 : 0);
    for (size_t i = 0; i < p.in_val.size(); ++i) {
        const Val &v = p.vals[p.in_val[i]];
        Tensor t;
        if (v.var.is_data()) {
            t = v.var.origin->data;
            if (!t.defined()) return ctx.fail(SAGE_ERR_INVALID, "a data variable of the program holds no tensor");
            sage_status st = t.to_device(ctx);
            if (st) return st;
        } else if (!fetch(v.var, &t)) {
            return ctx.fail(SAGE_ERR_INVALID, "internal: row program input not available");
        }
        if (t.data->planes_only) return ctx.fail(SAGE_ERR_INVALID, "internal: row program input exists as tf32 planes only");
        const bool aligned = p.vec == 1 || v.cls != Full || reinterpret_cast<uintptr_t>(t.ptr()) % 16 == 0;
        if (v.bcast_leaf) {
            if (t.desc.shape.strides != v.var.desc.shape.strides) return ctx.fail(SAGE_ERR_INVALID, "internal: a broadcast view arrived with other strides");
        } else if (!t.desc.shape.has_default_strides() || !aligned) {  // a strided view: gather it into a contiguous buffer first
            Tensor c;
            sage_status st = Tensor::uninit(ctx, t.desc, &c);
            if (st) return st;
            st = k::strided_copy(ctx, (const uint32_t *)t.ptr(), t.dims(), (uint32_t *)c.ptr(), c.desc.shape.strides.data());
            if (st) return st;
            t = c;
        }
        keep.push_back(t);
        pb[2 + i] = (uint64_t)reinterpret_cast<uintptr_t>(t.ptr());
    }
    std::vector<Tensor> &outs = *outs_;
    outs.assign(p.out_val.size(), Tensor());
    for (size_t i = 0; i < p.out_val.size(); ++i) {
        sage_status st = Tensor::uninit(ctx, p.vals[p.out_val[i]].var.desc, &outs[i]);
        if (st) return st;
        pb[2 + nin + i] = (uint64_t)reinterpret_cast<uintptr_t>(outs[i].ptr());
        const Val &ov = p.vals[p.out_val[i]];
        if (planes && i < planes->size() && (*planes)[i] && ov.cls == Full && ov.dtype == SAGE_F32) {
            st = storage_planes_attach(ctx, *outs[i].data);
            if (st) return st;
            pb[2 + nin + nout + i] = (uint64_t)reinterpret_cast<uintptr_t>(outs[i].data->split->planes.planes + outs[i].desc.shape.offset);
            pb[2 + nin + 2 * nout + i] = (uint64_t)outs[i].data->split->plane;
        }
    }
    const long long resident = (long long)ctx.sm_count * p.resident;  // persistent: as many blocks as fit at once
    const uint32_t grid[3] = {(uint32_t)std::min<long long>(p.rows, resident), 1, 1};
    const uint32_t block[3] = {(uint32_t)p.threads, 1, 1};
    void *params[1] = {pb.data()};
    return ctx.launch(p.module, "sage_row_program", grid, block, p.stage_bytes, params, nullptr, true);
}

}  // namespace sage
