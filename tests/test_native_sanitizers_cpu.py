"""The host-side native code under AddressSanitizer and UndefinedBehaviorSanitizer: the AutoPipe
partitioner (``csrc/autopipe.cpp``) is compiled with ``-fsanitize=address,undefined`` into a small
driver that replays the recorded cost vectors plus randomised and degenerate ones; any
out-of-bounds access, leak or undefined operation aborts the driver.  (Device code has no such
tool on this machine; its checks are the small / odd-shape tests against CPU references, the bounded
waits that report through a status word, and the two-rank skewed-arrival test.)"""
import os
import shutil
import subprocess
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "merak_b200", "csrc", "autopipe.cpp")

DRIVER = textwrap.dedent(r"""
    #include <cstdio>
    #include <cstdlib>
    #include <vector>
    extern "C" int mrk_autopipe_partition(const long long* fwd, const long long* bwd, int n, int stages, int* out);
    extern "C" long long mrk_autopipe_simulate(const long long* fwd, const long long* bwd, int n, const int* starts,
                                               int stages, int* critical);
    static int check(std::vector<long long> f, std::vector<long long> b, int stages, std::vector<int> want) {
      std::vector<int> out(stages, -1);
      int rc = mrk_autopipe_partition(f.data(), b.data(), (int)f.size(), stages, out.data());
      if (rc != 0) { std::printf("rc %d\n", rc); return 1; }
      if (!want.empty() && out != want) { std::printf("mismatch\n"); return 1; }
      for (int s = 1; s < stages; ++s) if (out[s] < out[s - 1]) { std::printf("not monotone\n"); return 1; }
      int critical = -7;
      long long t = mrk_autopipe_simulate(f.data(), b.data(), (int)f.size(), out.data(), stages, &critical);
      if (t < -1 || critical < -1 || critical >= stages) { std::printf("bad simulation result\n"); return 1; }
      return 0;
    }
    int main() {
      int bad = 0;
      std::vector<long long> f24(24, 1000), b24(24, 3000);
      bad += check(f24, b24, 4, {0, 6, 12, 18});
      bad += check(f24, b24, 2, {0, 12});
      std::vector<long long> f27 = {50};
      for (int i = 0; i < 12; ++i) { f27.push_back(100); f27.push_back(200); }
      f27.push_back(30); f27.push_back(400);
      std::vector<long long> b27;
      for (auto v : f27) b27.push_back(3 * v);
      bad += check(f27, b27, 4, {0, 8, 15, 21});
      bad += check(f27, b27, 8, {0, 4, 8, 12, 16, 19, 22, 25});
      bad += check({5, 5, 5, 5}, {5, 5, 5, 5}, 4, {0, 1, 2, 3});
      bad += check({1, 1, 100, 1, 1, 1}, {2, 2, 200, 2, 2, 2}, 3, {0, 2, 3});
      // degenerate and random inputs: one stage, as many stages as layers, zero costs, large costs
      bad += check({7}, {9}, 1, {0});
      bad += check({3, 3, 3}, {1, 1, 1}, 3, {});
      bad += check({0, 0, 0, 0, 0, 0}, {0, 0, 0, 0, 0, 0}, 2, {});
      unsigned s = 12345u;
      for (int rep = 0; rep < 40; ++rep) {
        int n = 2 + (int)((s = s * 1664525u + 1013904223u) >> 24) % 40;
        int stages = 1 + (int)((s = s * 1664525u + 1013904223u) >> 24) % (n < 8 ? n : 8);
        std::vector<long long> f(n), b(n);
        for (int i = 0; i < n; ++i) {
          f[i] = 1 + ((s = s * 1664525u + 1013904223u) >> 12) % 100000;
          b[i] = 1 + ((s = s * 1664525u + 1013904223u) >> 12) % 300000;
        }
        bad += check(f, b, stages, {});
      }
      std::printf("checked, %d bad\n", bad);
      return bad ? 1 : 0;
    }
""")


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_autopipe_under_asan_and_ubsan(tmp_path):
    drv = tmp_path / "driver.cpp"
    drv.write_text(DRIVER)
    exe = str(tmp_path / "autopipe_san")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
                            "-fno-omit-frame-pointer", SRC, str(drv), "-o", exe], capture_output=True, text=True)
    if build.returncode != 0 and ("cannot find" in build.stderr or "asan" in build.stderr.lower()):
        pytest.skip("sanitizer runtime not installed: " + build.stderr.splitlines()[-1])
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1"))
    assert run.returncode == 0, (run.stdout[-2000:], run.stderr[-3000:])
    assert "checked, 0 bad" in run.stdout
