"""CPU unit test of the per-device set-up caches (csrc/per_device.h): function attributes and occupancy results are kept
per CUDA device, so the "already done" state must be keyed by device ordinal and safe to use from several host threads."""
import os
import subprocess
import tempfile

from conftest import ROOT

PROGRAM = r"""
#include <cstdio>
#include <thread>
#include <vector>
#include "per_device.h"
using namespace amv;
#define CHECK(c) do { if (!(c)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #c); return 1; } } while (0)
int main() {
    PerDeviceOnce once;
    int calls[4] = {0, 0, 0, 0};
    // first use on device 0 runs the set-up; the second does not
    CHECK(once.run_once(0, [&] { ++calls[0]; return true; }));
    CHECK(once.run_once(0, [&] { ++calls[0]; return true; }));
    CHECK(calls[0] == 1 && once.is_done(0) && !once.is_done(1));
    // a second device has its own state
    CHECK(once.run_once(1, [&] { ++calls[1]; return true; }));
    CHECK(calls[1] == 1 && once.is_done(1));
    // a failed set-up is not remembered
    CHECK(!once.run_once(2, [&] { ++calls[2]; return false; }));
    CHECK(!once.is_done(2));
    CHECK(once.run_once(2, [&] { ++calls[2]; return true; }));
    CHECK(calls[2] == 2 && once.is_done(2));
    // ordinals outside the table are never cached
    CHECK(once.run_once(-1, [&] { ++calls[3]; return true; }));
    CHECK(once.run_once(kMaxDeviceOrdinals, [&] { ++calls[3]; return true; }));
    CHECK(once.run_once(-1, [&] { ++calls[3]; return true; }));
    CHECK(calls[3] == 3);
    // many threads, one set-up per device
    PerDeviceOnce shared;
    int runs[8] = {};
    std::vector<std::thread> th;
    for (int t = 0; t < 16; ++t)
        th.emplace_back([&, t] { for (int i = 0; i < 1000; ++i) shared.run_once(t % 8, [&] { ++runs[t % 8]; return true; }); });
    for (auto& x : th) x.join();
    for (int d = 0; d < 8; ++d) CHECK(runs[d] == 1);

    PerDeviceMemo memo;
    int v = 0;
    CHECK(!memo.get(0, 1000, &v));
    memo.put(0, 1000, 74);
    CHECK(memo.get(0, 1000, &v) && v == 74);
    CHECK(!memo.get(0, 2000, &v));      // another shared-memory size: not the cached answer
    CHECK(!memo.get(1, 1000, &v));      // another device: not the cached answer
    memo.put(1, 1000, 66);
    CHECK(memo.get(1, 1000, &v) && v == 66);
    CHECK(memo.get(0, 1000, &v) && v == 74);
    memo.put(0, 2000, 37);              // a new key replaces the device's entry
    CHECK(memo.get(0, 2000, &v) && v == 37 && !memo.get(0, 1000, &v));
    CHECK(!memo.get(-1, 1, &v) && !memo.get(kMaxDeviceOrdinals, 1, &v));
    std::printf("ok\n");
    return 0;
}
"""


def test_per_device_once_and_memo_are_keyed_by_device():
    with tempfile.TemporaryDirectory() as td:
        src, exe = os.path.join(td, "t.cpp"), os.path.join(td, "t")
        open(src, "w").write(PROGRAM)
        subprocess.run(["/usr/bin/g++", "-std=c++17", "-O1", "-pthread", "-I",
                        os.path.join(ROOT, "ameva-compute_b200", "csrc"), src, "-o", exe], check=True)
        out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stdout + out.stderr
