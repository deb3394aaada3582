// Stream-ordered caching allocator.  Policy follows src/session/memory.rs of the reference
// (cited per function); bookkeeping is in bytes.
#include <algorithm>
#include <cassert>

#include "runtime.h"

namespace sage {

Allocator::Allocator(std::unique_ptr<DeviceMem> mem, uint64_t capacity, bool use_cache)
    : mem_(std::move(mem)), capacity_(capacity), use_cache_(use_cache) {}

Allocator::~Allocator() {
    // Walk every segment from its head block and hand it back.
    std::vector<Block *> heads;
    auto collect = [&](FreeSet &s) {
        for (Block *b : s)
            if (!b->prev) heads.push_back(b);
    };
    collect(small_free_);
    collect(large_free_);
    // Only segments whose blocks are all free are returned here.  A segment with a block still in use belongs to a
    // tensor handle that outlives the context (Storage keeps the allocator alive through a shared_ptr, so this
    // destructor normally runs after the last such handle is gone); should one remain, its segment is deliberately
    // left to the process exit rather than freed under a live pointer.
    for (Block *h : heads) {
        bool all_free = true;
        for (Block *b = h; b; b = b->next) all_free &= b->free_;
        if (!all_free) continue;
        mem_->release(h->segment);
        for (Block *b = h; b;) {
            Block *n = b->next;
            delete b;
            b = n;
        }
    }
}

size_t Allocator::round_size(size_t bytes) {
    if (bytes == 0) bytes = 1;
    return (bytes + kMinBlock - 1) / kMinBlock * kMinBlock;
}

// Pool::get_free_block — memory.rs:283-334: best fit among blocks that are large enough,
// never carving a small request out of a >= 40 MiB block, nor a huge request out of a block
// more than 20 MiB larger; split off the remainder when it is worth keeping.
void Allocator::enter(FreeSet &pool, Block *b) {
    b->entered = searches_[&pool == &small_free_ ? 1 : 0];  // age 0: ages count the searches a block sits through
    pool.insert(b);
}

Block *Allocator::find_free(FreeSet &pool, size_t size) {
    ++searches_[&pool == &small_free_ ? 1 : 0];  // every block of the pool grows one search older (memory.rs:287)
    Block key;
    key.size = size;
    key.ptr = nullptr;
    auto it = pool.lower_bound(&key);
    for (; it != pool.end(); ++it) {
        Block *b = *it;
        if (size < kSplitLim && b->size >= kSplitLim) return nullptr;  // sorted: all later ones too
        if (size >= kSplitLim && b->size > size + kLargeBuffer) return nullptr;
        pool.erase(it);
        size_t rem = b->size - size;
        bool split = b->small ? (rem >= kMinBlock) : (size < kSplitLim && rem > kSmallSize);
        if (split) {
            Block *r = new Block();
            r->ptr = b->ptr + size;
            r->size = rem;
            r->small = b->small;
            r->segment = b->segment;
            r->prev = b;
            r->next = b->next;
            if (b->next) b->next->prev = r;
            b->next = r;
            b->size = size;
            enter(pool, r);
        }
        b->free_ = false;
        return b;
    }
    return nullptr;
}

// Pool::expand / alloc_size — memory.rs:246-281: 2 MiB segments for small requests, 20 MiB for
// requests under 10 MiB, otherwise the request rounded up to 2 MiB; refused when it would pass
// the capacity.
bool Allocator::grow(size_t size, bool small) {
    size_t seg = small ? kSmallBuffer
                       : (size < kMinLargeAlloc ? kLargeBuffer : (size + kRoundLarge - 1) / kRoundLarge * kRoundLarge);
    if (total_ + seg > capacity_) {
        oom_needed = total_ + seg - capacity_;
        oom_total = total_;
        return false;
    }
    void *p = mem_->alloc(seg);
    if (!p) {
        oom_needed = seg;
        oom_total = total_;
        return false;
    }
    ++device_allocs_;
    total_ += seg;
    peak_ = std::max(peak_, total_);
    Block *b = new Block();
    b->ptr = static_cast<char *>(p);
    b->size = seg;
    b->small = small;
    b->segment = p;
    enter(small ? small_free_ : large_free_, b);
    return true;
}

// Pool::alloc — memory.rs:336-363.
Block *Allocator::alloc(size_t bytes) {
    size_t size = round_size(bytes);
    if (!use_cache_) {
        // The reference's shipped configuration (context.rs:49): one device buffer per tensor.
        if (total_ + size > capacity_) {
            oom_needed = total_ + size - capacity_;
            oom_total = total_;
            return nullptr;
        }
        void *p = mem_->alloc(size);
        if (!p) {
            oom_needed = size;
            oom_total = total_;
            return nullptr;
        }
        ++device_allocs_;
        total_ += size;
        used_ += size;
        peak_ = std::max(peak_, total_);
        Block *b = new Block();
        b->ptr = static_cast<char *>(p);
        b->size = size;
        b->segment = p;
        b->free_ = false;
        return b;
    }
    bool small = size < kSmallSize;
    FreeSet &pool = small ? small_free_ : large_free_;
    Block *b = find_free(pool, size);
    if (!b) {
        garbage_collect();  // memory.rs:339: old cached segments go first, when the pool is nearly full
        if (!grow(size, small)) {
            release_largest(size);  // memory.rs:344-349: give cached segments back, largest first, then retry
            if (!grow(size, small)) {
                release_cached();  // (not in the reference) everything that is cached, small pool included
                if (!grow(size, small)) return nullptr;
            }
        }
        b = find_free(pool, size);
        if (!b) return nullptr;
    }
    used_ += b->size;
    return b;
}

// Pool::free — memory.rs:365-408: merge with free neighbours of the same segment.
void Allocator::free(Block *b) {
    if (!b) return;
    if (!use_cache_) {
        used_ -= b->size;
        total_ -= b->size;
        mem_->release(b->segment);
        delete b;
        return;
    }
    used_ -= b->size;
    FreeSet &pool = b->small ? small_free_ : large_free_;
    b->free_ = true;
    if (b->prev && b->prev->free_) {
        Block *p = b->prev;
        pool.erase(p);
        p->size += b->size;
        p->next = b->next;
        if (b->next) b->next->prev = p;
        delete b;
        b = p;
    }
    if (b->next && b->next->free_) {
        Block *n = b->next;
        pool.erase(n);
        b->size += n->size;
        b->next = n->next;
        if (n->next) n->next->prev = b;
        delete n;
    }
    enter(pool, b);
}

// Pool::garbage_collect — memory.rs:410-452.  Runs only when 80 % of the capacity is in use; frees whole
// cached segments of the large pool, oldest first (age >= the average age of what is left), until 20 % of
// the capacity has been given back or nothing old enough remains.
size_t Allocator::garbage_collect() {
    const uint64_t threshold = (uint64_t)((double)capacity_ * 0.8);  // GC_THRESHOLD
    if (used_ < threshold) return 0;
    const uint64_t target = capacity_ - threshold;
    const uint64_t now = searches_[0];
    uint64_t total_age = 0, freeable = 0;
    for (Block *b : large_free_)
        if (!b->prev && !b->next) {
            total_age += now - b->entered;
            ++freeable;
        }
    size_t reclaimed = 0;
    bool freed = true;
    while (reclaimed < target && freed && freeable > 0) {
        const uint64_t age_threshold = total_age / freeable;
        freed = false;
        for (auto it = large_free_.begin(); it != large_free_.end();) {
            Block *b = *it;
            if (!b->prev && !b->next && now - b->entered >= age_threshold) {
                it = large_free_.erase(it);
                reclaimed += b->size;
                total_age -= now - b->entered;
                --freeable;
                total_ -= b->size;
                mem_->release(b->segment);
                delete b;
                freed = true;
            } else {
                ++it;
            }
        }
    }
    if (reclaimed) {
        ++gc_runs;
        gc_reclaimed += reclaimed;
    }
    return reclaimed;
}

// Pool::release_cached_blocks — memory.rs:454-474: whole cached segments of the large pool, largest first,
// until max(size, SPLIT_LIM) bytes have gone back to the device.
size_t Allocator::release_largest(size_t size) {
    size_t released = 0;
    const size_t want = std::max(size, kSplitLim);
    while (released < want) {
        Block *best = nullptr;
        for (auto it = large_free_.rbegin(); it != large_free_.rend(); ++it)
            if (!(*it)->prev && !(*it)->next) {
                best = *it;  // the set is ordered by size: the first whole segment from the top is the largest
                break;
            }
        if (!best) break;
        large_free_.erase(best);
        released += best->size;
        total_ -= best->size;
        mem_->release(best->segment);
        delete best;
    }
    return released;
}

// Every unsplit free segment of both pools (sage_release_cached, and the last resort of alloc).
void Allocator::release_cached() {
    for (FreeSet *pool : {&small_free_, &large_free_}) {
        for (auto it = pool->begin(); it != pool->end();) {
            Block *b = *it;
            if (!b->prev && !b->next) {
                it = pool->erase(it);
                total_ -= b->size;
                mem_->release(b->segment);
                delete b;
            } else {
                ++it;
            }
        }
    }
}

}  // namespace sage
