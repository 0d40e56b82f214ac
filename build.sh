#!/usr/bin/env bash
# Build driver. The reference's build.sh offers packaging, sanitizer, coverage and test switches
# (reference: build.sh:684-725,753-884); these are the ones that apply to this tree.
#   ./build.sh                 library + torch extension (sm_100a), in-tree under hccl_b200/lib
#   ./build.sh --debug         extra library with device-side bounds checks  (hccl_b200/lib/libhccl_b200_debug.so)
#   ./build.sh --asan          extra library with AddressSanitizer on host code (libhccl_b200_asan.so); run the CPU tests on it with
#                              LD_PRELOAD="$(gcc -print-file-name=libasan.so) $(gcc -print-file-name=libstdc++.so.6)" ASAN_OPTIONS=detect_leaks=0 \
#                              HCCL_B200_LIB=hccl_b200/lib/libhccl_b200_asan.so python -m pytest tests -m "not gpu"
#   ./build.sh --examples      also build examples/bin/*
#   ./build.sh --test          run the CPU test-suite afterwards
#   ./build.sh --pkg           dist/hccl_b200-<version>-sm100a.tar.gz
#   ./build.sh --ptxas         print registers / spills / shared memory of every kernel
#   ./build.sh --clean         remove build directories and built libraries
set -euo pipefail
cd "$(dirname "$0")"
PY=${PYTHON:-python}
DEBUG=0 ASAN=0 EX=0 TEST=0 PKG=0 PTXAS=0 CLEAN=0
for a in "$@"; do
  case "$a" in
    --debug) DEBUG=1 ;; --asan) ASAN=1 ;; --examples) EX=1 ;; --test|-u) TEST=1 ;; --pkg) PKG=1 ;; --ptxas) PTXAS=1 ;; --clean) CLEAN=1 ;;
    -h|--help) sed -n 2,15p "$0"; exit 0 ;;
    *) echo "unknown option $a" >&2; exit 2 ;;
  esac
done
if [ $CLEAN = 1 ]; then rm -rf build build_debug build_asan dist examples/bin; rm -f hccl_b200/lib/*.so; echo cleaned; exit 0; fi
if [ $PTXAS = 1 ]; then
  $PY -c "from hccl_b200.utils import build; build.build_native(verbose=True, ptxas_info=True, flavor='ptxas')" | grep -E "ptxas info|Compiling entry|registers" || true
  rm -f hccl_b200/lib/libhccl_b200_ptxas.so
fi
$PY -m hccl_b200.utils.build
[ $DEBUG = 1 ] && $PY -m hccl_b200.utils.build --flavor=debug
[ $ASAN = 1 ] && $PY -m hccl_b200.utils.build --flavor=asan
[ $EX = 1 ] && make -C examples -j8
[ $PKG = 1 ] && $PY -c "from hccl_b200.utils import build; print('package:', build.package())"
[ $TEST = 1 ] && $PY -m pytest tests -x -q -m "not gpu"
echo "done"
