// One-time set-up state that CUDA keeps per device (function attributes such as the dynamic shared-memory limit, occupancy
// results), cached per device ordinal: a process may hold contexts on several GPUs, and a host may launch from several
// threads. Plain C++ (no CUDA types) so that the keying can be unit-tested on a machine without a GPU.
#pragma once
#include <mutex>
#include <stdint.h>

namespace amv {

constexpr int kMaxDeviceOrdinals = 64;

// A set of "done on this device" flags. run_once(dev, fn) calls fn() under the lock the first time it is asked for
// `dev` and remembers a true result; a false result (set-up failed) is not remembered, so the next call tries again.
// Ordinals outside [0, kMaxDeviceOrdinals) are never cached: fn runs every time.
class PerDeviceOnce {
public:
    template <typename Fn>
    bool run_once(int dev, Fn&& fn) {
        if (dev < 0 || dev >= kMaxDeviceOrdinals) return fn();
        std::lock_guard<std::mutex> lock(mu_);
        if (done_ & (1ull << dev)) return true;
        if (!fn()) return false;
        done_ |= 1ull << dev;
        return true;
    }
    bool is_done(int dev) {
        if (dev < 0 || dev >= kMaxDeviceOrdinals) return false;
        std::lock_guard<std::mutex> lock(mu_);
        return (done_ >> dev) & 1ull;
    }

private:
    std::mutex mu_;
    uint64_t done_ = 0;
};

// A small per-device memo of one integer result keyed by one integer argument (the occupancy of a kernel for a given
// dynamic shared-memory size): get() returns false until put() has stored a value for the same (device, key).
class PerDeviceMemo {
public:
    bool get(int dev, uint32_t key, int* value) {
        if (dev < 0 || dev >= kMaxDeviceOrdinals) return false;
        std::lock_guard<std::mutex> lock(mu_);
        if (!valid_[dev] || key_[dev] != key) return false;
        *value = value_[dev];
        return true;
    }
    void put(int dev, uint32_t key, int value) {
        if (dev < 0 || dev >= kMaxDeviceOrdinals) return;
        std::lock_guard<std::mutex> lock(mu_);
        valid_[dev] = true;
        key_[dev] = key;
        value_[dev] = value;
    }

private:
    std::mutex mu_;
    bool valid_[kMaxDeviceOrdinals] = {};
    uint32_t key_[kMaxDeviceOrdinals] = {};
    int value_[kMaxDeviceOrdinals] = {};
};

}  // namespace amv
