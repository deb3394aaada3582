// CUDA C emitter for fused elementwise maps.
//
// Reference: compile_map (src/ops/map.rs:369-410) writes one OpenCL kernel per (expression, input
// strides, input offsets): `y[gid] = expr(x_k[idx_k])`, with each idx_k either `offset + gid` or an
// ndim-step div/mul loop whose strides are literals in the source (src/ops/core.rs:113-175).
// Here:
//   * strides, extents and offsets are kernel PARAMETERS, so one compiled kernel serves every
//     tensor with the same access pattern (the source text is the cache key, as in the reference's
//     Context::get_program, but it no longer changes with the shape);
//   * axes are collapsed before emission (unit axes dropped, axes that form one run for every
//     operand merged), so the common cases need 0-2 integer divisions per element instead of ndim;
//   * when the innermost collapsed axis is unit-stride or broadcast for every operand, each thread
//     handles 4 consecutive elements with 128-bit loads and stores.
#include "map_emit.h"

#include <cstdio>
#include <sstream>

namespace sage {

static const char *kPrelude = R"(
typedef unsigned int uint;
#define SG __device__ __forceinline__
SG float sg_abs(float x) { return fabsf(x); }
SG int sg_abs(int x) { return x < 0 ? -x : x; }
SG uint sg_abs(uint x) { return x; }
SG float sg_log(float x) { return logf(x); }
SG float sg_exp(float x) { return expf(x); }
SG float sg_sqrt(float x) { return sqrtf(x); }
SG float sg_erf(float x) { return erff(x); }
SG float sg_ceil(float x) { return ceilf(x); }
SG float sg_floor(float x) { return floorf(x); }
SG float sg_round(float x) { return roundf(x); }
SG float sg_sin(float x) { return sinf(x); }
SG float sg_sinh(float x) { return sinhf(x); }
SG float sg_cos(float x) { return cosf(x); }
SG float sg_cosh(float x) { return coshf(x); }
SG float sg_tan(float x) { return tanf(x); }
SG float sg_tanh(float x) { return tanhf(x); }
SG float sg_asin(float x) { return asinf(x); }
SG float sg_asinh(float x) { return asinhf(x); }
SG float sg_acos(float x) { return acosf(x); }
SG float sg_acosh(float x) { return acoshf(x); }
SG float sg_atan(float x) { return atanf(x); }
SG float sg_atanh(float x) { return atanhf(x); }
SG float sg_square(float x) { return x * x; }
SG int sg_square(int x) { return x * x; }
SG uint sg_square(uint x) { return x * x; }
SG float sg_recip(float x) { return 1.0f / x; }
SG int sg_recip(int x) { return 1 / x; }
SG uint sg_recip(uint x) { return 1u / x; }
SG float sg_sign(float x) { return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : (x == x ? x : 0.0f)); }
SG int sg_sign(int x) { return (x > 0) - (x < 0); }
SG uint sg_sign(uint x) { return x > 0u; }
SG float sg_pow(float a, float b) { return powf(a, b); }
SG float sg_mod(float a, float b) { return fmodf(a, b); }
SG int sg_mod(int a, int b) { return a % b; }
SG uint sg_mod(uint a, uint b) { return a % b; }
SG float sg_min(float a, float b) { return fminf(a, b); }
SG int sg_min(int a, int b) { return a < b ? a : b; }
SG uint sg_min(uint a, uint b) { return a < b ? a : b; }
SG float sg_max(float a, float b) { return fmaxf(a, b); }
SG int sg_max(int a, int b) { return a > b ? a : b; }
SG uint sg_max(uint a, uint b) { return a > b ? a : b; }
SG float sg_lit(uint bits) { return __uint_as_float(bits); }
// hi = x rounded to tf32 (nearest, ties away), lo = x - hi; when the rounding overflows or x is inf / nan,
// hi is the truncated value and lo what is left of a finite x (the rule of the GEMM's own split pass)
SG void sg_split_tf32(float x, float *hi, float *lo) {
  const uint xb = __float_as_uint(x);
  const uint hb = (xb + 0x1000u) & 0xffffe000u;  // cvt.rna.tf32.f32 of a finite value, as an add and a mask
  const bool finite = (xb & 0x7f800000u) != 0x7f800000u;
  const bool overflow = !finite || (hb & 0x7f800000u) == 0x7f800000u;
  const float hf = __uint_as_float(overflow ? (xb & 0xffffe000u) : hb);
  *hi = hf;
  *lo = finite ? x - hf : 0.f;
}
)";

const char *map_prelude_text() { return kPrelude; }

static const char *ctype(int dt) { return dt == SAGE_F32 ? "float" : dt == SAGE_I32 ? "int" : "uint"; }
static const char *vtype(int dt) { return dt == SAGE_F32 ? "float4" : dt == SAGE_I32 ? "int4" : "uint4"; }

sage_status map_plan(const std::string &expr, const std::vector<MapOperand> &in, int out_dtype, const void *y,
                     int out_ndim, const long long *out_ext, MapPlan *plan, bool emit_source, bool planes) {
    const int nin = (int)in.size();
    // ---- collapse axes
    long long ext[k::kMaxDims];
    std::vector<std::vector<long long>> str(nin);
    int nd = 0;
    long long n = 1;
    for (int i = 0; i < out_ndim; ++i) {
        n *= out_ext[i];
        if (out_ext[i] == 1) continue;
        bool merge = nd > 0;
        if (merge)
            for (int q = 0; q < nin; ++q)
                if (str[q][nd - 1] != in[q].view.str[i] * out_ext[i]) merge = false;
        if (merge) {
            ext[nd - 1] *= out_ext[i];
            for (int q = 0; q < nin; ++q) str[q][nd - 1] = in[q].view.str[i];
        } else {
            ext[nd] = out_ext[i];
            for (int q = 0; q < nin; ++q) str[q].push_back(in[q].view.str[i]);
            ++nd;
        }
    }
    if (nd == 0) {
        ext[0] = 1;
        for (int q = 0; q < nin; ++q) str[q].push_back(0);
        nd = 1;
    }
    plan->n = n;
    plan->ndim = nd;
    for (int i = 0; i < nd; ++i) plan->ext[i] = (unsigned long long)ext[i];
    plan->strides = str;

    // ---- classify operands: D direct (idx = g), S scalar broadcast, G generic strided
    std::string modes;
    std::vector<long long> dflt(nd);
    {
        long long s = 1;
        for (int i = nd - 1; i >= 0; --i) {
            dflt[i] = s;
            s *= ext[i];
        }
    }
    bool vec_ok = (ext[nd - 1] % 4 == 0) && (reinterpret_cast<uintptr_t>(y) % 16 == 0);
    for (int q = 0; q < nin; ++q) {
        bool direct = true, scalar = true;
        for (int i = 0; i < nd; ++i) {
            if (str[q][i] != dflt[i]) direct = false;
            if (str[q][i] != 0) scalar = false;
        }
        if (n == 1) direct = true;
        char m = direct ? 'D' : scalar ? 'S' : 'G';
        const bool aligned = reinterpret_cast<uintptr_t>(in[q].ptr) % 16 == 0;
        if (m == 'D' && !aligned) vec_ok = false;
        if (m == 'G') {
            const long long inner = str[q][nd - 1];
            if (inner == 1) {
                m = 'G';  // unit inner stride: vector load possible
                if (!aligned) vec_ok = false;
                for (int i = 0; i < nd - 1; ++i)
                    if (str[q][i] % 4 != 0) vec_ok = false;
            } else if (inner == 0) {
                m = 'B';  // broadcast along the inner axis: one scalar load per 4 outputs
            } else {
                m = 'X';  // arbitrary inner stride: scalar path only
                vec_ok = false;
            }
        }
        modes.push_back(m);
    }
    const int vec = vec_ok ? 4 : 1;
    plan->vec = vec;
    const bool wide = n >= (1LL << 32);
    const char *it = wide ? "unsigned long long" : "unsigned int";
    plan->signature = modes + ":" + std::to_string(vec) + ":" + std::to_string(nd) + (wide ? "w" : "n") + (planes ? "P" : "");
    if (!emit_source) return SAGE_OK;  // the caller already holds the kernel for this signature

    // ---- emit
    std::ostringstream s;
    s << kPrelude;
    s << "struct MapP { long long n; unsigned long long ext[" << k::kMaxDims << "]; long long str["
      << (nin > 0 ? nin : 1) << "][" << k::kMaxDims << "]; };\n";
    s << "SG " << ctype(out_dtype) << " sage_expr(";
    for (int q = 0; q < nin; ++q) s << (q ? ", " : "") << ctype(in[q].dtype) << " x" << q;
    s << ") { return (" << ctype(out_dtype) << ")(" << expr << "); }\n";
    s << "extern \"C\" __global__ void __launch_bounds__(256) sage_map(";
    for (int q = 0; q < nin; ++q) s << "const " << ctype(in[q].dtype) << " *__restrict__ x" << q << "_buf, ";
    s << ctype(out_dtype) << " *__restrict__ y, const MapP p" << (planes ? ", float *__restrict__ hi, const long long plane" : "") << ") {\n";
    // launched as a programmatic dependent: wait for the kernel before this one before touching memory
    s << "  asm volatile(\"griddepcontrol.launch_dependents;\" ::: \"memory\");\n";
    s << "  asm volatile(\"griddepcontrol.wait;\" ::: \"memory\");\n";
    s << "  const " << it << " q = (" << it << ")blockIdx.x * blockDim.x + threadIdx.x;\n";
    s << "  const " << it << " g = q * " << vec << ";\n";
    s << "  if (g >= (" << it << ")p.n) return;\n";
    bool need_coords = false;
    for (char m : modes)
        if (m == 'G' || m == 'B' || m == 'X') need_coords = true;
    if (need_coords) {
        for (int q = 0; q < nin; ++q)
            if (modes[q] != 'D' && modes[q] != 'S') s << "  long long i" << q << " = 0;\n";
        s << "  { " << it << " rem = g, c;\n";
        for (int d = nd - 1; d >= 0; --d) {
            if (d == 0)
                s << "    c = rem;\n";
            else
                s << "    c = rem % (" << it << ")p.ext[" << d << "]; rem /= (" << it << ")p.ext[" << d << "];\n";
            for (int q = 0; q < nin; ++q)
                if (modes[q] != 'D' && modes[q] != 'S') s << "    i" << q << " += (long long)c * p.str[" << q << "][" << d << "];\n";
        }
        s << "  }\n";
    }
    if (vec == 1) {
        for (int q = 0; q < nin; ++q) {
            s << "  const " << ctype(in[q].dtype) << " x" << q << " = x" << q << "_buf[";
            if (modes[q] == 'D') s << "g";
            else if (modes[q] == 'S') s << "0";
            else s << "i" << q;
            s << "];\n";
        }
        s << "  const " << ctype(out_dtype) << " r = sage_expr(";
        for (int q = 0; q < nin; ++q) s << (q ? ", " : "") << "x" << q;
        s << ");\n  y[g] = r;\n";
        if (planes) s << "  { float h, l; sg_split_tf32(r, &h, &l); hi[g] = h; hi[plane + g] = l; }\n";
    } else {
        for (int q = 0; q < nin; ++q) {
            const char *ct = ctype(in[q].dtype);
            if (modes[q] == 'D' || modes[q] == 'G') {
                s << "  const " << vtype(in[q].dtype) << " v" << q << " = *reinterpret_cast<const " << vtype(in[q].dtype)
                  << " *>(x" << q << "_buf + " << (modes[q] == 'D' ? std::string("g") : "i" + std::to_string(q)) << ");\n";
                s << "  const " << ct << " a" << q << "[4] = {v" << q << ".x, v" << q << ".y, v" << q << ".z, v" << q << ".w};\n";
            } else {
                s << "  const " << ct << " s" << q << " = x" << q << "_buf[" << (modes[q] == 'S' ? std::string("0") : "i" + std::to_string(q))
                  << "];\n";
                s << "  const " << ct << " a" << q << "[4] = {s" << q << ", s" << q << ", s" << q << ", s" << q << "};\n";
            }
        }
        s << "  " << vtype(out_dtype) << " r;\n";
        const char *comp[4] = {"x", "y", "z", "w"};
        for (int e = 0; e < 4; ++e) {
            s << "  r." << comp[e] << " = sage_expr(";
            for (int q = 0; q < nin; ++q) s << (q ? ", " : "") << "a" << q << "[" << e << "]";
            s << ");\n";
        }
        s << "  *reinterpret_cast<" << vtype(out_dtype) << " *>(y + g) = r;\n";
        if (planes)
            s << "  { float4 h, l; sg_split_tf32(r.x, &h.x, &l.x); sg_split_tf32(r.y, &h.y, &l.y); sg_split_tf32(r.z, &h.z, &l.z); "
                 "sg_split_tf32(r.w, &h.w, &l.w);\n    *reinterpret_cast<float4 *>(hi + g) = h; *reinterpret_cast<float4 *>(hi + plane + g) = l; }\n";
    }
    s << "}\n";
    plan->source = s.str();
    return SAGE_OK;
}

struct MapPHost {
    long long n;
    unsigned long long ext[k::kMaxDims];
};

sage_status map_launch(Context &ctx, const std::string &expr, const std::vector<MapOperand> &in, int out_dtype,
                       void *y, int out_ndim, const long long *out_ext, MapCache *cache, float *hi, long long plane) {
    const bool planes = hi != nullptr && out_dtype == SAGE_F32;
    MapPlan plan;
    sage_status st = map_plan(expr, in, out_dtype, y, out_ndim, out_ext, &plan, false, planes);
    if (st) return st;
    if (plan.n == 0) return SAGE_OK;
    Module *mod = nullptr;
    if (cache && cache->owner == &ctx) {
        auto it = cache->by_signature.find(plan.signature);
        if (it != cache->by_signature.end()) mod = it->second;
    }
    if (!mod) {
        st = map_plan(expr, in, out_dtype, y, out_ndim, out_ext, &plan, true, planes);  // first use: write the source
        if (st) return st;
        st = ctx.module_get(plan.source, &mod);
        if (st) return st;
        if (cache) {
            if (cache->owner != &ctx) {
                cache->by_signature.clear();
                cache->owner = &ctx;
            }
            cache->by_signature[plan.signature] = mod;
        }
    }
    const int nin = (int)in.size();
    // by-value parameter block: n, ext[8], str[nin][8]
    std::vector<long long> pb(1 + k::kMaxDims + (size_t)(nin > 0 ? nin : 1) * k::kMaxDims, 0);
    pb[0] = plan.n;
    for (int i = 0; i < plan.ndim; ++i) pb[1 + i] = (long long)plan.ext[i];
    for (int q = 0; q < nin; ++q)
        for (int i = 0; i < plan.ndim; ++i) pb[1 + k::kMaxDims + (size_t)q * k::kMaxDims + i] = plan.strides[q][i];
    std::vector<const void *> ptrs(nin);
    std::vector<void *> params;
    for (int q = 0; q < nin; ++q) {
        ptrs[q] = in[q].ptr;
        params.push_back(&ptrs[q]);
    }
    params.push_back(&y);
    params.push_back(pb.data());
    if (planes) {
        params.push_back(&hi);
        params.push_back(&plane);
    }
    const long long chunks = (plan.n + plan.vec - 1) / plan.vec;
    const uint32_t grid[3] = {(uint32_t)((chunks + 255) / 256), 1, 1};
    const uint32_t block[3] = {256, 1, 1};
    std::string label;
    if (ctx.verbose_names) {
        label = "map{" + expr + "}n=" + std::to_string(plan.n) + ",v" + std::to_string(plan.vec) + "," + plan.signature;
        for (char &ch : label)
            if (ch == ' ') ch = '_';
    }
    return ctx.launch(mod, "sage_map", grid, block, 0, params.data(), label.empty() ? nullptr : label.c_str(), true);
}

}  // namespace sage
