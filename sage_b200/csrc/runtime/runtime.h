// Runtime under the C ABI: context (device + in-order stream), stream-ordered caching
// allocator, NVRTC module cache, launch bookkeeping.  Replaces the reference's
// src/session/device.rs, src/session/memory.rs and the cache half of
// src/session/context.rs.
#pragma once
#include <cstdint>
#include <list>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../../include/sage_cuda.h"

struct CUmod_st;
struct CUfunc_st;
typedef struct CUstream_st *cudaStream_t;

namespace sage {

// ------------------------------------------------------------------------------------------
// Allocator: restates the pool policy of src/session/memory.rs (size classes :23-43, best fit
// + split :283-334, merge on free :365-408, release-cached :454-474) in bytes instead of 4-byte
// elements, with the merge defect fixed (merged size is the sum), and reuse ordered by the
// context's single stream: a block freed after kernel k was enqueued may be handed to kernel
// k+1 without a synchronisation because both run in stream order.
// ------------------------------------------------------------------------------------------
struct DeviceMem {  // where segments come from: cudaMalloc, or fake addresses on a planning context
    virtual ~DeviceMem() {}
    virtual void *alloc(size_t bytes) = 0;  // nullptr on failure
    virtual void release(void *p) = 0;
};

struct Block {
    char *ptr = nullptr;
    size_t size = 0;
    bool free_ = true;
    bool small = false;
    Block *prev = nullptr, *next = nullptr;  // neighbours inside the same segment
    void *segment = nullptr;
    uint64_t entered = 0;  // the pool's search count when the block last entered its free list (Age, memory.rs:756-786)
};

class Allocator {
public:
    static constexpr size_t kMinBlock = 512;                // MIN_BLOCK_SIZE 128 elements
    static constexpr size_t kSmallSize = 1u << 20;          // SMALL_SIZE
    static constexpr size_t kSmallBuffer = 2u << 20;        // SMALL_BUFFER
    static constexpr size_t kLargeBuffer = 20u << 20;       // LARGE_BUFFER
    static constexpr size_t kMinLargeAlloc = 10u << 20;     // MIN_LARGE_ALLOC
    static constexpr size_t kRoundLarge = 2u << 20;         // ROUND_LARGE
    static constexpr size_t kSplitLim = 2 * kLargeBuffer;   // SPLIT_LIM

    Allocator(std::unique_ptr<DeviceMem> mem, uint64_t capacity, bool use_cache);
    ~Allocator();

    // Returns nullptr on out-of-memory and fills needed/total like MemoryError::OutOfMemory.
    Block *alloc(size_t bytes);
    void free(Block *b);
    void release_cached();
    // Pool::garbage_collect — memory.rs:410-452; returns the bytes given back to the device.
    size_t garbage_collect();
    uint64_t gc_runs = 0, gc_reclaimed = 0;  // collections that freed something, bytes they freed

    uint64_t capacity() const { return capacity_; }
    uint64_t mem_total() const { return total_; }
    uint64_t mem_used() const { return used_; }
    uint64_t mem_peak() const { return peak_; }
    uint64_t num_device_allocs() const { return device_allocs_; }
    uint64_t oom_needed = 0, oom_total = 0;

private:
    struct Cmp {
        bool operator()(const Block *a, const Block *b) const {
            return a->size != b->size ? a->size < b->size : a->ptr < b->ptr;
        }
    };
    typedef std::set<Block *, Cmp> FreeSet;
    Block *find_free(FreeSet &pool, size_t size);
    bool grow(size_t size, bool small);
    size_t release_largest(size_t size);
    void enter(FreeSet &pool, Block *b);
    uint64_t searches_[2] = {0, 0};  // get_free_block calls per pool (large, small): the clock block ages are read against
    static size_t round_size(size_t bytes);

    std::unique_ptr<DeviceMem> mem_;
    uint64_t capacity_, total_ = 0, used_ = 0, peak_ = 0, device_allocs_ = 0;
    bool use_cache_;
    FreeSet small_free_, large_free_;
};

// ------------------------------------------------------------------------------------------
struct Module {
    std::string source;
    std::vector<char> cubin;
    CUmod_st *cu_module = nullptr;  // null on a planning context
    std::unordered_map<std::string, CUfunc_st *> functions;
};

class Context {
public:
    static sage_status create(int device, const sage_ctx_opts &opts, Context **out);
    ~Context();

    int device() const { return device_; }
    // Makes this context's GPU the calling thread's current device (kernel launches, attribute calls and
    // cudaMalloc act on the current device, whatever stream they are given).  Every C-ABI entry point calls it, so
    // a process may hold contexts on several GPUs, or change its device between calls.
    void make_current() const;
    bool dry() const { return device_ < 0; }
    cudaStream_t stream() const { return stream_; }
    const sage_ctx_opts &opts() const { return opts_; }
    Allocator &allocator() { return *alloc_; }
    // Tensors keep the allocator alive past the context, so a handle dropped late still returns
    // its block to a live object.
    std::shared_ptr<Allocator> allocator_ptr() { return alloc_; }

    sage_status fail(sage_status code, const std::string &msg) {
        last_error_ = msg;
        return code;
    }
    const std::string &last_error() const { return last_error_; }
    sage_status check_cuda(int err, const char *what);

    sage_status module_get(const std::string &src, Module **out);
    // A launcher whose translation unit is a fixed text behind a few generated lines looks its module up under those
    // lines alone (hashing and comparing the whole source on every launch costs the host ~10 us per launch).
    Module *module_find(const std::string &key) const {
        auto it = module_keys_.find(key);
        return it == module_keys_.end() ? nullptr : it->second;
    }
    void module_remember(const std::string &key, Module *m) { module_keys_[key] = m; }
    // How many blocks of `block_threads` threads and `smem` dynamic bytes of this kernel fit on one SM (>= 1).
    int blocks_per_sm(Module *m, const char *name, int block_threads, uint32_t smem);
    // `dependent`: the kernel begins with griddepcontrol.wait, so it may be launched with programmatic
    // stream serialisation (its prologue overlaps the tail of the kernel before it).
    sage_status launch(Module *m, const char *name, const uint32_t grid[3], const uint32_t block[3],
                       uint32_t smem, void **params, const char *label = nullptr, bool dependent = false, int cluster = 1);
    // Programmatic dependent launch for the library's own kernels that wait on the grid dependency
    // themselves (GEMM, row kernels, generated maps).  Off with SAGE_PDL=0.
    bool pdl = true;
    // When set, JIT-compiled map kernels are recorded under "map{<expression>}" instead of
    // "sage_map" in traces and profiles (more names, same launches).
    bool verbose_names = false;

    // bookkeeping for every kernel the library launches itself (static kernels call note_launch)
    void note_launch(const char *name) {
        ++kernel_launches;
        if (tracing) trace.append(name).push_back('\n');
        if (profiling) profile_mark(name);
    }
    void note_memset() { ++memset_launches; }
    uint64_t kernel_launches = 0, memset_launches = 0;
    bool tracing = false;
    std::string trace;

    // Per-kernel device timing: a CUDA event is recorded on the stream in front of every launch;
    // on an in-order stream the time between two consecutive events is the time the earlier
    // launch took (plus any gap before the next one was enqueued).
    bool profiling = false;
    void profile_begin();
    void profile_mark(const char *name);
    // "name launches total_ms\n" per kernel name, sorted by total time; stops profiling.
    std::string profile_end();

    void *timer_events[2] = {nullptr, nullptr};  // cudaEvent_t pair of sage_timer_start/stop
    uint32_t *status_word_dev = nullptr;  // device word kernels OR error bits into (word 0 of a 4 KiB block)
    // Ticket counters for kernels whose last block finishes the work of the others (column reductions): zero between
    // launches, each launch leaves them zero.  Launches of one context are ordered on its stream, so they can share them.
    static constexpr int kTickets = 960;
    unsigned *tickets() const { return reinterpret_cast<unsigned *>(status_word_dev) + 64; }
    // Scratch of the stream-K GEMM (partial accumulators of tiles shared between CTAs + their hand-over flags), taken
    // from the pool on first use and kept; `streamk_epoch` is the value the flags of the next launch are raised to.
    Block *streamk_block = nullptr;
    Block *gemm_trace_block = nullptr;  // per-CTA cycle counters of a GEMM launch run with SAGE_GEMM_TRACE (sm_count x 16 words)
    size_t streamk_bytes = 0;
    uint32_t streamk_epoch = 0;
    // Set by the evaluator around one operator's compute(): a tensor-core GEMM will read the result,
    // so a producer that can should also write the tf32 hi/lo planes of what it computes.
    bool hint_emit_planes = false;
    // ... and nothing else reads it: the producer may skip the fp32 store and write only the planes.
    bool hint_planes_only = false;
    int sm_count = 148;

private:
    Context() {}
    int device_ = -1;
    cudaStream_t stream_ = nullptr;
    sage_ctx_opts opts_{};
    std::shared_ptr<Allocator> alloc_;
    std::string last_error_;
    std::unordered_map<std::string, std::unique_ptr<Module>> modules_;
    std::unordered_map<std::string, Module *> module_keys_;  // short keys of modules_ entries (which own them)
    std::vector<void *> prof_events_;  // cudaEvent_t pool, reused across profile runs
    std::vector<std::string> prof_names_;
    size_t prof_used_ = 0;
};

}  // namespace sage

// The opaque handles of the C ABI.
struct sage_ctx {
    sage::Context *impl;
};
struct sage_buf {
    sage::Block *block;
    void *ptr;
    size_t size;
    sage::Context *owner;
};
struct sage_module {
    sage::Module *impl;
};
