// The cache of captured step graphs and its memory policy: Graphs / GraphCache of the reference's host
// (src/cuda/core.rs:1105-1252), restated. One graph per step shape; the keys are many (row counts, key splits, MTP
// steps, adapter steps) and the driver keeps a dropped graph's memory for the next ones, so the cache is bounded:
// unbounded until less than `floor` bytes of device memory are free when a new graph is about to be captured, then
// capped at what it holds, lowered by a sixteenth whenever the free memory falls further; the least recently used
// graphs go. A capture that runs out of memory lowers the cap to three quarters of what is held, and that step runs
// without a graph (the same kernels, the same results). Pure bookkeeping: every CUDA call goes through the hooks, so
// the policy runs on a CPU with fakes behind them.
#pragma once
#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <vector>

namespace qb {

template <class K, class G>
class GraphCache {
  public:
    struct Hooks {
        std::function<size_t()> free_mem;              // free device memory now
        std::function<void(G&)> destroy;               // drop a graph
        std::function<void()> sync;                    // the graphs about to go may still run
        std::function<size_t(size_t)> release;         // give `bytes` of the cache pool back to the driver (may be null)
    };
    static constexpr size_t NO_CAP = (size_t)-1;

    GraphCache(Hooks h, size_t floor_bytes) : hooks_(std::move(h)), floor_(floor_bytes) {}
    ~GraphCache() { clear(); }

    // the graph of `key`, marked as just used; null when there is none
    G* find(const K& key) {
        tick_++;
        auto it = graphs_.find(key);
        if (it == graphs_.end()) return nullptr;
        it->second.second = tick_;
        return &it->second.first;
    }

    // Before a capture: room for one more graph within the cap (make_room, core.rs:1198-1233)
    void make_room() {
        const size_t free = hooks_.free_mem();
        if (free < std::min(floor_, low_) && !graphs_.empty()) {
            const size_t n = std::min(cap_, graphs_.size());
            cap_ = cap_ == NO_CAP ? n : n - n / 16;
            low_ = free;
        }
        if (graphs_.size() >= cap_) {
            cap_ = std::max<size_t>(cap_, 1);
            evict();
        }
        if (free < floor_ / 2 && hooks_.release) hooks_.release(floor_ - free);
    }

    void insert(const K& key, G g) { graphs_[key] = std::make_pair(std::move(g), tick_); }

    // A capture found no memory: fewer graphs from now on (core.rs:1180-1192)
    void on_out_of_memory() {
        cap_ = graphs_.size() * 3 / 4;
        evict();
    }

    // drop the graphs whose keys `keep` refuses (their kernels' arguments changed; retain, core.rs:1146-1148)
    void retain(const std::function<bool(const K&)>& keep) {
        bool synced = false;
        for (auto it = graphs_.begin(); it != graphs_.end();) {
            if (keep(it->first)) { ++it; continue; }
            if (!synced) { hooks_.sync(); synced = true; }
            hooks_.destroy(it->second.first);
            it = graphs_.erase(it);
        }
    }
    void clear() { retain([](const K&) { return false; }); }

    size_t size() const { return graphs_.size(); }
    size_t cap() const { return cap_; }
    bool holds(const K& key) const { return graphs_.count(key) != 0; }

  private:
    // the least recently used graphs go until fewer than the cap are kept (evict, core.rs:1235-1250)
    void evict() {
        if (graphs_.size() < cap_) return;
        hooks_.sync();
        std::vector<std::pair<uint64_t, K>> by_age;
        for (auto& g : graphs_) by_age.emplace_back(g.second.second, g.first);
        std::sort(by_age.begin(), by_age.end(), [](const auto& a, const auto& b) { return a.first < b.first; });
        const size_t n = graphs_.size() + 1 - std::max<size_t>(cap_, 1);
        for (size_t i = 0; i < n && i < by_age.size(); i++) {
            auto it = graphs_.find(by_age[i].second);
            hooks_.destroy(it->second.first);
            graphs_.erase(it);
        }
    }

    Hooks hooks_;
    size_t floor_;
    std::map<K, std::pair<G, uint64_t>> graphs_;
    uint64_t tick_ = 0;
    size_t cap_ = NO_CAP, low_ = (size_t)-1;
};

}  // namespace qb
