// What one kernel instantiation has to remember about a device between launches: that its dynamic
// shared-memory limit has been raised, and how many blocks of a given size fit on an SM.
//
// The limit is raised ONCE per device, to the largest size any launch of the instantiation can ask
// for, and never lowered again - a launch shape that needs little must not take the opt-in away from
// a later launch that needs a lot.  Lookups are serialised by a mutex, so handles driven by
// different host threads can share an instantiation.  The CUDA calls come in as callables, which
// keeps this header free of CUDA and lets a host-only test exercise the logic.
#pragma once
#include <cstddef>
#include <map>
#include <mutex>
#include <utility>

namespace mascot {

class LaunchCache {
public:
    // `raise_limit(bytes)` sets the instantiation's dynamic shared-memory limit on the current device,
    // `blocks_per_sm(block, smem, &fit)` asks how many blocks of that shape an SM holds; both return 0
    // on success.  Returns 0 and the cached or freshly queried answer in *fit, or the callable's error.
    template <class Raise, class Query>
    int lookup(int device, int block_threads, size_t smem_block, size_t smem_max, Raise raise_limit, Query blocks_per_sm, int* fit) {
        std::lock_guard<std::mutex> lock(mu_);
        Device& d = devices_[device];
        if (!d.limit_raised) {
            const int rc = raise_limit(smem_max);
            if (rc != 0) return rc;
            d.limit_raised = true;
        }
        const std::pair<int, size_t> key(block_threads, smem_block);
        auto it = d.fit.find(key);
        if (it == d.fit.end()) {
            int f = 0;
            const int rc = blocks_per_sm(block_threads, smem_block, &f);
            if (rc != 0) return rc;
            it = d.fit.emplace(key, f).first;
        }
        *fit = it->second;
        return 0;
    }

private:
    struct Device {
        bool limit_raised = false;
        std::map<std::pair<int, size_t>, int> fit;
    };
    std::mutex mu_;
    std::map<int, Device> devices_;
};

}  // namespace mascot
