// Activation memory of a step: liveness intervals packed into one arena, planned once per capacity bucket.
//
// The reference plans every graph build: liveness over the topological order, then best-fit-decreasing placement into
// one arena with 256-byte alignment (src/internal/graph_compiler.cpp:147-191 liveness, :286-398 placement: sort by size,
// then lifetime, then birth; candidate offsets are 0 and the ends of placed buffers that are alive at the same time), and
// reports peak bytes, buffers, reuse and bytes saved (include/velomind/graph.h:40-46).
//
// Here the parts ask for and give back buffers while a step runs.  The first step of a capacity bucket records that
// sequence (with ordinary allocations); the plan made from it serves every later step of the bucket from one arena, with
// no allocation.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <set>

#include "ops.h"

namespace vmb {

namespace {
constexpr size_t ALIGN = 256;
size_t aligned(size_t n) { return (std::max<size_t>(n, 1) + ALIGN - 1) / ALIGN * ALIGN; }
}  // namespace

ArenaPlan plan_arena(const std::vector<Interval>& intervals) {
    const size_t n = intervals.size();
    ArenaPlan plan;
    plan.sizes.resize(n);
    plan.offsets.assign(n, 0);
    for (size_t i = 0; i < n; ++i) plan.sizes[i] = aligned(intervals[i].bytes);
    std::vector<size_t> order(n);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
        if (plan.sizes[a] != plan.sizes[b]) return plan.sizes[a] > plan.sizes[b];
        const int la = intervals[a].death - intervals[a].birth, lb = intervals[b].death - intervals[b].birth;
        if (la != lb) return la > lb;
        return intervals[a].birth < intervals[b].birth;
    });
    std::vector<size_t> placed;
    for (size_t i : order) {
        std::vector<size_t> rivals;              // placed buffers that are alive at the same time
        for (size_t j : placed)
            if (!(intervals[j].death < intervals[i].birth || intervals[i].death < intervals[j].birth)) rivals.push_back(j);
        std::set<size_t> candidates{0};
        for (size_t j : rivals) candidates.insert(plan.offsets[j] + plan.sizes[j]);
        for (size_t c : candidates) {            // the end of the highest rival always fits
            bool free_here = true;
            for (size_t j : rivals)
                if (!(c + plan.sizes[i] <= plan.offsets[j] || plan.offsets[j] + plan.sizes[j] <= c)) { free_here = false; break; }
            if (free_here) { plan.offsets[i] = c; break; }
        }
        for (size_t j : placed) {                // bytes that an earlier buffer, dead meanwhile, used too
            if (std::find(rivals.begin(), rivals.end(), j) != rivals.end()) continue;
            if (plan.offsets[j] < plan.offsets[i] + plan.sizes[i] && plan.offsets[i] < plan.offsets[j] + plan.sizes[j]) { ++plan.reused_count; break; }
        }
        placed.push_back(i);
    }
    size_t total = 0;
    for (size_t i = 0; i < n; ++i) {
        plan.peak_bytes = std::max(plan.peak_bytes, plan.offsets[i] + plan.sizes[i]);
        total += plan.sizes[i];
    }
    plan.buffer_count = static_cast<int>(n);
    plan.bytes_saved = static_cast<long long>(total) - static_cast<long long>(plan.peak_bytes);
    return plan;
}

Workspace::Workspace(bool poison_) : poison(poison_) {
    // host-side fault injection (the reference's VELOMIND_FAIL_GRAPH_BUILD_AFTER_ALLOCATIONS, graph_compiler.cpp:562-569): the
    // N-th buffer a step asks for is refused; the step is abandoned and can be run again
    const char* env = std::getenv("VELOMIND_B200_FAIL_STEP_AFTER_BUFFERS");
    if (env && *env && std::all_of(env, env + std::strlen(env), [](char c) { return c >= '0' && c <= '9'; })) fail_after = std::atoll(env);
}

Workspace::~Workspace() = default;

bool Workspace::planned(const std::string& bucket) const {
    auto it = plans_.find(bucket);
    return it != plans_.end() && arena_ && arena_->bytes >= it->second.peak_bytes;
}

const ArenaPlan* Workspace::plan(const std::string& bucket) const {
    auto it = plans_.find(bucket);
    return it == plans_.end() ? nullptr : &it->second;
}

void Workspace::begin(const std::string& bucket, cudaStream_t stream) {
    if (open_) throw Error("Workspace::begin: the previous step was not ended");
    open_ = true;
    key_ = bucket;
    stream_ = stream;
    recording_ = !planned(bucket);
    log_.clear();
    live_.clear();
    clock_ = 0;
    next_ = 0;
}

void* Workspace::take(size_t bytes) {
    if (!open_) throw Error("Workspace::take outside of a step");
    const int idx = next_;
    if (fail_after >= 0 && idx >= fail_after)
        throw Error(format("injected failure: buffer %d of the step was refused (fail_after = %lld)", idx, fail_after));
    ++next_;
    ++clock_;
    void* p = nullptr;
    if (recording_) {
        loose_.push_back(std::make_unique<DeviceBuffer>(aligned(bytes)));
        p = loose_.back()->ptr;
        log_.push_back(Interval{bytes, clock_, clock_});
    } else {
        const ArenaPlan& plan = plans_.at(key_);
        if (idx >= plan.buffer_count || aligned(bytes) != plan.sizes[idx])
            throw Error(format("Workspace: a step of bucket %s asks for other buffers than the one it was planned from", key_.c_str()));
        p = static_cast<char*>(arena_->ptr) + plan.offsets[idx];
    }
    live_[p] = Live{idx, bytes};
    // (debugging aid, with the poisoning of freed buffers: a buffer starts as NaN too, so that a kernel which leaves part of its
    //  output unwritten shows in the step's result whatever the memory held before)
    if (poison && bytes) ops::cuda_check(cudaMemsetAsync(p, 0xff, bytes, stream_), "poisoning a fresh buffer");
    return p;
}

void Workspace::give(void* p) {
    if (!p) return;
    auto it = live_.find(p);
    if (it == live_.end()) throw Error("Workspace::give: this buffer was not taken in this step (or given twice)");
    const Live l = it->second;
    live_.erase(it);
    ++clock_;
    if (recording_) log_[l.index].death = clock_;
    if (poison && l.bytes) {
        // whoever reads the buffer after this point (a part that gave it back too early, a kernel still to run on it) now reads
        // NaN (all bits set: a NaN as float32 and as bfloat16, -1 as an integer), and the step's result shows it
        ops::cuda_check(cudaMemsetAsync(p, 0xff, l.bytes, stream_), "poisoning a freed buffer");
    }
}

void Workspace::end() {
    if (!open_) return;
    if (recording_) {
        for (const auto& kv : live_) log_[kv.second.index].death = clock_ + 1;     // still held: alive to the step's end
        ArenaPlan plan = plan_arena(log_);
        // the recording step's own buffers may still be read by kernels in flight: wait before they are freed
        ops::cuda_check(cudaStreamSynchronize(stream_), "ending a recorded step");
        loose_.clear();
        if (!arena_ || arena_->bytes < plan.peak_bytes) {
            arena_.reset();
            arena_ = std::make_unique<DeviceBuffer>(plan.peak_bytes);
            ++generation;
        }
        plans_[key_] = std::move(plan);
    }
    open_ = false;
    live_.clear();
}

void Workspace::abort() {
    if (recording_ && stream_) cudaStreamSynchronize(stream_);
    loose_.clear();
    open_ = false;
    live_.clear();
}

}  // namespace vmb
