"""B200-native speculative-decoding decode step behind the reference engine's API.

The directory name has a hyphen, so it is imported through `load_package()` below (or by
putting it on `sys.modules` under the name `silicon_violetto_b200`, which is what
`__graft_entry__`, `bench.py` and the tests do).

  vlt      the .vlt weight container and int8 quantiser (numpy)
  synth    random-init weight files for the benchmark configurations
  build    compiles csrc/ into libvioletto_b200.so with nvcc for sm_100a
  engine   ctypes mirror of the reference's `Engine` / `Generator` API over the C ABI
"""
PACKAGE_NAME = "silicon_violetto_b200"
