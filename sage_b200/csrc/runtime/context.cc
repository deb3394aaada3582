// Context: device + one in-order stream + allocator + JIT module cache.
// Reference counterparts: Device::new (src/session/device.rs:45-71), Context::with_device
// (src/session/context.rs:43-52), KernelProgram::new (device.rs:201-213),
// Context::get_program_with_id (context.rs:62-83), Kernel::launch (device.rs:297-318).
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nvrtc.h>
#include <sys/stat.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>

#include "runtime.h"

namespace sage {

// ---- driver API, resolved lazily so the library also loads on a machine without a GPU driver
typedef int (*PFN_cuModuleLoadData)(CUmod_st **, const void *);
typedef int (*PFN_cuModuleUnload)(CUmod_st *);
typedef int (*PFN_cuModuleGetFunction)(CUfunc_st **, CUmod_st *, const char *);
typedef int (*PFN_cuLaunchKernel)(CUfunc_st *, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                                  cudaStream_t, void **, void **);
typedef int (*PFN_cuFuncSetAttribute)(CUfunc_st *, int, int);
typedef CUresult (*PFN_cuLaunchKernelEx)(const CUlaunchConfig *, CUfunction, void **, void **);
typedef int (*PFN_cuGetErrorString)(int, const char **);

struct Driver {
    void *lib = nullptr;
    PFN_cuModuleLoadData ModuleLoadData = nullptr;
    PFN_cuModuleUnload ModuleUnload = nullptr;
    PFN_cuModuleGetFunction ModuleGetFunction = nullptr;
    PFN_cuLaunchKernel LaunchKernel = nullptr;
    PFN_cuLaunchKernelEx LaunchKernelEx = nullptr;
    PFN_cuFuncSetAttribute FuncSetAttribute = nullptr;
    PFN_cuGetErrorString GetErrorString = nullptr;
    bool ok = false;
};

static Driver &driver() {
    static Driver d;
    if (!d.lib) {
        d.lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        if (d.lib) {
            d.ModuleLoadData = (PFN_cuModuleLoadData)dlsym(d.lib, "cuModuleLoadData");
            d.ModuleUnload = (PFN_cuModuleUnload)dlsym(d.lib, "cuModuleUnload");
            d.ModuleGetFunction = (PFN_cuModuleGetFunction)dlsym(d.lib, "cuModuleGetFunction");
            d.LaunchKernel = (PFN_cuLaunchKernel)dlsym(d.lib, "cuLaunchKernel");
            d.LaunchKernelEx = (PFN_cuLaunchKernelEx)dlsym(d.lib, "cuLaunchKernelEx");
            d.FuncSetAttribute = (PFN_cuFuncSetAttribute)dlsym(d.lib, "cuFuncSetAttribute");
            d.GetErrorString = (PFN_cuGetErrorString)dlsym(d.lib, "cuGetErrorString");
            d.ok = d.ModuleLoadData && d.ModuleGetFunction && d.LaunchKernel;
        }
    }
    return d;
}

void *driver_symbol(const char *name) {  // used by the TMA descriptor code
    Driver &d = driver();
    return d.lib ? dlsym(d.lib, name) : nullptr;
}

static std::string cu_err(int e) {
    const char *s = nullptr;
    if (driver().GetErrorString) driver().GetErrorString(e, &s);
    return std::string(s ? s : "unknown driver error") + " (" + std::to_string(e) + ")";
}

// ---- device memory sources
struct CudaMem : DeviceMem {
    void *alloc(size_t bytes) override {
        void *p = nullptr;
        if (cudaMalloc(&p, bytes) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        return p;
    }
    void release(void *p) override { cudaFree(p); }
};

// Planning contexts hand out addresses from a counter; they are never dereferenced.
struct FakeMem : DeviceMem {
    uintptr_t next = 0x100000000ull;
    void *alloc(size_t bytes) override {
        void *p = reinterpret_cast<void *>(next);
        next += (bytes + 4095) / 4096 * 4096;
        return p;
    }
    void release(void *) override {}
};

sage_status Context::check_cuda(int err, const char *what) {
    if (err == cudaSuccess) return SAGE_OK;
    return fail(SAGE_ERR_DEVICE, std::string(what) + ": " + cudaGetErrorString((cudaError_t)err));
}

sage_status Context::create(int device, const sage_ctx_opts &opts, Context **out) {
    std::unique_ptr<Context> c(new Context());
    c->opts_ = opts;
    c->device_ = device;
    if (const char *e = getenv("SAGE_REF_COMPAT")) c->opts_.ref_compat = atoi(e);
    if (const char *e = getenv("SAGE_PATTERN_FUSION")) c->opts_.pattern_fusion = atoi(e);
    if (const char *e = getenv("SAGE_GEMM_BACKEND")) c->opts_.gemm_backend = atoi(e);
    if (const char *e = getenv("SAGE_VERBOSE_NAMES")) c->verbose_names = atoi(e) != 0;
    if (const char *e = getenv("SAGE_PDL")) c->pdl = atoi(e) != 0;
    uint64_t cap = opts.mem_capacity_bytes;
    if (const char *e = getenv("SAGE_MEM_CAP")) cap = strtoull(e, nullptr, 10);
    if (device < 0) {
        if (!cap) cap = 160ull << 30;
        c->alloc_.reset(new Allocator(std::unique_ptr<DeviceMem>(new FakeMem()), cap, opts.use_cache != 0));
        *out = c.release();
        return SAGE_OK;
    }
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device >= n) {
        cudaGetLastError();
        return SAGE_ERR_NO_DEVICE;
    }
    if (cudaSetDevice(device) != cudaSuccess) return SAGE_ERR_DEVICE;
    if (cudaFree(0) != cudaSuccess) return SAGE_ERR_DEVICE;
    if (cudaStreamCreateWithFlags(&c->stream_, cudaStreamNonBlocking) != cudaSuccess) return SAGE_ERR_DEVICE;
    cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device);
    if (!cap) {
        size_t free_b = 0, total_b = 0;
        cudaMemGetInfo(&free_b, &total_b);
        cap = (uint64_t)(free_b * 0.9);
    }
    c->alloc_.reset(new Allocator(std::unique_ptr<DeviceMem>(new CudaMem()), cap, opts.use_cache != 0));
    if (cudaMalloc(&c->status_word_dev, 4096) != cudaSuccess) return SAGE_ERR_DEVICE;
    cudaMemsetAsync(c->status_word_dev, 0, 4096, c->stream_);
    *out = c.release();
    return SAGE_OK;
}

void Context::make_current() const {
    if (dry()) return;
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != device_) cudaSetDevice(device_);
}

Context::~Context() {
    if (!dry()) {
        cudaSetDevice(device_);
        cudaStreamSynchronize(stream_);
        for (auto &kv : modules_)
            if (kv.second->cu_module && driver().ModuleUnload) driver().ModuleUnload(kv.second->cu_module);
        if (streamk_block) alloc_->free(streamk_block);
        streamk_block = nullptr;
        if (gemm_trace_block) alloc_->free(gemm_trace_block);
        gemm_trace_block = nullptr;
        alloc_.reset();
        if (status_word_dev) cudaFree(status_word_dev);
        cudaStreamDestroy(stream_);
    }
}

// ---- JIT: NVRTC to an sm_100a cubin, cached in memory by source text and on disk by hash
static uint64_t fnv1a(const std::string &s, uint64_t h) {
    for (unsigned char ch : s) {
        h ^= ch;
        h *= 1099511628211ull;
    }
    return h;
}

static std::string cache_path(const std::string &src) {
    const char *dir = getenv("SAGE_JIT_CACHE_DIR");
    if (!dir || !*dir) return "";
    mkdir(dir, 0755);
    char name[64];
    snprintf(name, sizeof name, "/%016llx%016llx.cubin", (unsigned long long)fnv1a(src, 1469598103934665603ull),
             (unsigned long long)fnv1a(src, 0x9e3779b97f4a7c15ull));
    return std::string(dir) + name;
}

static bool nvrtc_compile(const std::string &src, std::vector<char> *cubin, std::string *log) {
    nvrtcProgram prog;
    if (nvrtcCreateProgram(&prog, src.c_str(), "sage_jit.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS) {
        *log = "nvrtcCreateProgram failed";
        return false;
    }
    const char *opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device", "--fmad=true"};
    nvrtcResult r = nvrtcCompileProgram(prog, 4, opts);
    size_t log_size = 0;
    nvrtcGetProgramLogSize(prog, &log_size);
    if (log_size > 1) {
        log->resize(log_size);
        nvrtcGetProgramLog(prog, &(*log)[0]);
    }
    if (r != NVRTC_SUCCESS) {
        nvrtcDestroyProgram(&prog);
        return false;
    }
    size_t n = 0;
    nvrtcGetCUBINSize(prog, &n);
    cubin->resize(n);
    nvrtcGetCUBIN(prog, cubin->data());
    nvrtcDestroyProgram(&prog);
    return true;
}

sage_status Context::module_get(const std::string &src, Module **out) {
    auto it = modules_.find(src);
    if (it != modules_.end()) {
        *out = it->second.get();
        return SAGE_OK;
    }
    std::unique_ptr<Module> m(new Module());
    m->source = src;
    std::string path = cache_path(src);
    if (!path.empty()) {
        std::ifstream f(path, std::ios::binary);
        if (f) m->cubin.assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
    }
    if (m->cubin.empty()) {
        std::string log;
        if (!nvrtc_compile(src, &m->cubin, &log)) return fail(SAGE_ERR_COMPILE, "NVRTC: " + log);
        if (!path.empty()) {
            std::ofstream f(path, std::ios::binary);
            f.write(m->cubin.data(), (std::streamsize)m->cubin.size());
        }
    }
    if (!dry()) {
        Driver &d = driver();
        if (!d.ok) return fail(SAGE_ERR_DEVICE, "libcuda.so.1 could not be loaded");
        cudaSetDevice(device_);
        int e = d.ModuleLoadData(&m->cu_module, m->cubin.data());
        if (e) return fail(SAGE_ERR_DEVICE, "cuModuleLoadData: " + cu_err(e));
    }
    *out = m.get();
    modules_[src] = std::move(m);
    return SAGE_OK;
}

int Context::blocks_per_sm(Module *m, const char *name, int block_threads, uint32_t smem) {
    if (dry()) return 1;
    Driver &d = driver();
    typedef int (*PFN_occupancy)(int *, CUfunc_st *, int, size_t);
    static PFN_occupancy occupancy = (PFN_occupancy)dlsym(d.lib, "cuOccupancyMaxActiveBlocksPerMultiprocessor");
    CUfunc_st *fn = nullptr;
    auto it = m->functions.find(name);
    if (it == m->functions.end()) {
        if (d.ModuleGetFunction(&fn, m->cu_module, name)) return 1;
        if (smem > 48 * 1024 && d.FuncSetAttribute) d.FuncSetAttribute(fn, 8 /*MAX_DYNAMIC_SHARED_SIZE_BYTES*/, (int)smem);
        m->functions[name] = fn;
    } else {
        fn = it->second;
    }
    int n = 0;
    if (!occupancy || occupancy(&n, fn, block_threads, smem) || n < 1) return 1;
    return n;
}

sage_status Context::launch(Module *m, const char *name, const uint32_t grid[3], const uint32_t block[3],
                            uint32_t smem, void **params, const char *label, bool dependent, int cluster) {
    note_launch(label && verbose_names ? label : name);
    if (dry()) return SAGE_OK;
    Driver &d = driver();
    CUfunc_st *fn = nullptr;
    auto it = m->functions.find(name);
    if (it == m->functions.end()) {
        int e = d.ModuleGetFunction(&fn, m->cu_module, name);
        if (e) return fail(SAGE_ERR_DEVICE, std::string("cuModuleGetFunction(") + name + "): " + cu_err(e));
        if (smem > 48 * 1024 && d.FuncSetAttribute) d.FuncSetAttribute(fn, 8 /*MAX_DYNAMIC_SHARED_SIZE_BYTES*/, (int)smem);
        m->functions[name] = fn;
    } else {
        fn = it->second;
    }
    if (grid[0] == 0 || grid[1] == 0 || grid[2] == 0) return SAGE_OK;
    int e;
    if (cluster > 1 && !d.LaunchKernelEx) return fail(SAGE_ERR_DEVICE, "cuLaunchKernelEx is not available for a cluster launch");
    if (((dependent && pdl) || cluster > 1) && d.LaunchKernelEx) {
        CUlaunchAttribute attr[2];
        memset(attr, 0, sizeof attr);
        unsigned nattr = 0;
        if (dependent && pdl) {
            attr[nattr].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
            attr[nattr].value.programmaticStreamSerializationAllowed = 1;
            ++nattr;
        }
        if (cluster > 1) {
            attr[nattr].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
            attr[nattr].value.clusterDim.x = (unsigned)cluster;
            attr[nattr].value.clusterDim.y = 1;
            attr[nattr].value.clusterDim.z = 1;
            ++nattr;
        }
        CUlaunchConfig cfg;
        memset(&cfg, 0, sizeof cfg);
        cfg.gridDimX = grid[0];
        cfg.gridDimY = grid[1];
        cfg.gridDimZ = grid[2];
        cfg.blockDimX = block[0];
        cfg.blockDimY = block[1];
        cfg.blockDimZ = block[2];
        cfg.sharedMemBytes = smem;
        cfg.hStream = stream_;
        cfg.attrs = attr;
        cfg.numAttrs = nattr;
        e = d.LaunchKernelEx(&cfg, fn, params, nullptr);
    } else {
        e = d.LaunchKernel(fn, grid[0], grid[1], grid[2], block[0], block[1], block[2], smem, stream_, params, nullptr);
    }
    if (e) return fail(SAGE_ERR_DEVICE, std::string("cuLaunchKernel(") + name + "): " + cu_err(e));
    return SAGE_OK;
}

// ---- per-kernel timing with events in front of every launch
void Context::profile_begin() {
    prof_used_ = 0;
    prof_names_.clear();
    profiling = !dry();
}

void Context::profile_mark(const char *name) {
    if (prof_used_ == prof_events_.size()) {
        cudaEvent_t ev;
        if (cudaEventCreate(&ev) != cudaSuccess) {
            profiling = false;
            return;
        }
        prof_events_.push_back(ev);
    }
    cudaEventRecord((cudaEvent_t)prof_events_[prof_used_++], stream_);
    prof_names_.push_back(name);
}

std::string Context::profile_end() {
    std::string out;
    if (!profiling) return out;
    profile_mark("");  // closing event
    profiling = false;
    cudaStreamSynchronize(stream_);
    std::map<std::string, std::pair<uint64_t, double>> acc;
    for (size_t i = 0; i + 1 < prof_used_; ++i) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, (cudaEvent_t)prof_events_[i], (cudaEvent_t)prof_events_[i + 1]);
        auto &a = acc[prof_names_[i]];
        a.first += 1;
        a.second += ms;
    }
    std::vector<std::pair<std::string, std::pair<uint64_t, double>>> rows(acc.begin(), acc.end());
    std::sort(rows.begin(), rows.end(), [](const auto &a, const auto &b) { return a.second.second > b.second.second; });
    char line[256];
    for (auto &r : rows) {
        snprintf(line, sizeof line, "%s %llu %.6f\n", r.first.c_str(), (unsigned long long)r.second.first, r.second.second);
        out += line;
    }
    return out;
}

}  // namespace sage
