"""CPU oracle for the DeepSeek-V4 attention prologue.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package; the shipped `flaggems_vllm` package never does.

* `c_oracle`   - ctypes front end of `dsv4_oracle.c` (plain C, OpenMP).
* `torch_path` - the same arithmetic stated with torch CPU tensor ops in the
                 order the upstream torch reference path uses; timed as the CPU
                 baseline.
* `ref_loader` - runs the upstream test file's own `ref_impl` where the upstream
                 tree is present (used to make and to check the golden vectors).
"""
