#!/bin/bash
# TEST INFRASTRUCTURE ONLY -- builds the unmodified reference library (Euler, AVX-512 + VNNI)
# straight from its sources with g++ so that the CPU restatement in this folder can be pinned
# against it and so that it can be timed as the CPU baseline.  Nothing the product ships or runs
# depends on anything produced here.
#
#   usage:  oracle/build_ref.sh [REFERENCE_ROOT]
#           (default: $EULER_REFERENCE, else a checkout named `reference` beside this repository)
#
# Outputs go to oracle/_ref/ only (git-ignored):
#   oracle/_ref/kgen/*.cpp     (O,T) function-table translation units (see below)
#   oracle/_ref/obj/*.o
#   oracle/_ref/libel.so       the reference library
#   oracle/_ref/libiomp5.so    the OpenMP runtime binary the reference bundles (copied, not built)
#   oracle/_ref/ref_driver     oracle/ref_driver.cpp linked against libel.so
#
# The reference's CMake project is NOT used.  Its only code-generation step -- six small shell
# functions under src/kernel/*_gen.sh that expand every DECL_*_TBL line of a "binder" header into
# one .cpp holding a table of template instantiations -- is invoked directly with the output
# directory pointed at oracle/_ref/kgen; the reference tree is never written.
#
# Flags follow cmake/flags.cmake (g++ branch) + WITH_VNNI.  Four additions are needed with g++ 13:
#   -mavx512vnni            flags.cmake forgets it for g++ even when WITH_VNNI is on
#   -include string/cstdint include/euler.hpp uses std::string / uint8_t without including them
#   -faligned-new           alignas(64) classes are new'ed under -std=c++11
#   -mf16c                  F16C intrinsics used by the half-precision variants
# and the int8 depthwise units are compiled with -include ref_gxx_unaligned.h (unaligned 64-byte
# moves where g++ would emit aligned ones; no arithmetic changes).
set -euo pipefail
HERE=$(cd "$(dirname "$0")" && pwd)
REF=${1:-${EULER_REFERENCE:-$(cd "$HERE/../.." && pwd)/reference}}
OUT=$HERE/_ref
JOBS=${JOBS:-$(nproc)}
CXX=${ORACLE_CXX:-$( [ -x /usr/bin/g++ ] && echo /usr/bin/g++ || echo g++ )}

if [ ! -d "$REF/src/kernel" ]; then
  echo "build_ref: reference tree not found at $REF -- keeping whatever is already in $OUT" >&2
  exit 0
fi
mkdir -p "$OUT/kgen" "$OUT/obj"

FLAGS="-std=c++11 -O2 -DNDEBUG -fopenmp -fPIC -fvisibility=hidden -w \
 -DWITH_VNNI -DMT_RUNTIME=MT_RUNTIME_OMP -DEULER_VERSION=oracle \
 -mavx512f -mavx512dq -mavx512bw -mavx512vl -mavx512vnni -mfma -mf16c \
 -include string -include cstdint -faligned-new \
 -I$REF -I$REF/include -I$REF/src -I$REF/tests -I$REF/src/common"

# 1. instantiation tables (idempotent: skipped when already present)
if [ ! -f "$OUT/kgen/.done" ]; then
  for fam in gemm u8s8_gemm conv u8s8_conv vmg_conv u8s8_depthwise_conv; do
    cp "$REF/src/kernel/elk_${fam}_binder.hxx" "$OUT/kgen/"
    (cd "$REF" && bash "$REF/src/kernel/elk_${fam}_gen.sh" \
        "$OUT/kgen/elk_${fam}_binder.hxx" "$OUT/kgen" "$CXX" OFF)
  done
  touch "$OUT/kgen/.done"
fi

# 2. compile every library source + every table TU, in parallel
SRCS=$(ls "$REF"/src/*.cpp "$REF"/src/common/el_log.cpp "$OUT"/kgen/*.cpp)
compile_one() {
  src=$1; obj="$OUT/obj/$(basename "${src%.cpp}").o"
  extra=""
  # the int8 depthwise units need unaligned 64-byte moves under g++ (see ref_gxx_unaligned.h)
  case "$(basename "$src")" in *depthwise*) extra="-include $HERE/ref_gxx_unaligned.h";; esac
  if [ ! -f "$obj" ] || [ "$src" -nt "$obj" ] || { [ -n "$extra" ] && [ "$HERE/ref_gxx_unaligned.h" -nt "$obj" ]; }; then
    $CXX $FLAGS $extra -c "$src" -o "$obj"
  fi
}
export -f compile_one; export OUT CXX FLAGS HERE
echo "$SRCS" | xargs -P "$JOBS" -I{} bash -c 'compile_one {}'

# 3. link
cp -f "$REF/lib/libiomp5.so" "$OUT/libiomp5.so"
$CXX -shared -o "$OUT/libel.so" "$OUT"/obj/*.o -L"$OUT" -liomp5 -lrt -Wl,-rpath,'$ORIGIN'

# 4. the driver used by tests / fixtures / the CPU-baseline leg of the bench
if [ -f "$HERE/ref_driver.cpp" ]; then
  $CXX -std=c++11 -O2 -include string -include cstdint -I"$REF/include" \
      "$HERE/ref_driver.cpp" -o "$OUT/ref_driver" -L"$OUT" -lel -liomp5 -Wl,-rpath,'$ORIGIN'
fi
echo "build_ref: done -> $OUT"
