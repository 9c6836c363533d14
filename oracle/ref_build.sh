#!/usr/bin/env bash
# Compiles the reference's own sources for the batched search path, where they lie in a reference
# checkout (read-only), into oracle/_ref/. Nothing is copied: the only files added are the stub
# for the five NVMe (BaM) symbols the path never reaches without an NVMe provider, and the driver
# that runs the reference API on an index directory and dumps its results (both in this folder).
# The reference's build system is not used (it needs a BaM submodule that is not vendored).
#   usage: ref_build.sh /path/to/reference
set -euo pipefail
REF="${1:-${TOPOANNS_REFERENCE:-}}"
if [[ -z "$REF" || ! -d "$REF" ]]; then
    echo "usage: ref_build.sh /path/to/reference (or set TOPOANNS_REFERENCE)" >&2
    exit 2
fi
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
mkdir -p "$OUT/obj"
NVCC="${NVCC:-nvcc}"
FLAGS=(-std=c++17 -O2 -gencode arch=compute_100a,code=sm_100a --expt-relaxed-constexpr -rdc=true
       -I"$REF/include" -I"$REF/src/search" -I"$REF/src/io" -Xcompiler -fPIC -w)
# RVQ entry selection: the definitions the reference's own build gives its RVQ support library
# (CMakeLists.txt:187-193); <cblas.h> comes from ref_shim/ (three training-only routines).
RVQ_FLAGS=(-I"$REF/src/legacy_rvq/gas_legacy/anns" -I"$HERE/ref_shim"
           -DANNS_SEARCH_DIM=128 -DANNS_RVQ_DISABLE_SEARCH_LOG -DUSE_L2_DIST_ -D_CUDA -D__CUDA__)
SRCS=(src/search/topology_search_kernel.cu src/search/pq_query_tables.cu src/search/rerank_exact.cu
      src/providers/pinned_topology.cu src/search/topology_search.cpp src/search/topoanns_search.cpp
      src/search/pq_distance_oracle.cpp src/search/search_resources.cpp src/search/entry_provider.cpp
      src/search/search_stop_condition.cpp src/search/rerank_reuse_profiler.cpp src/io/pq_index.cpp
      src/io/hpq_index.cpp src/io/topology_layout.cpp src/io/vector_page_layout.cpp
      src/io/vector_page_provider.cpp src/builder/vector_store_builder.cpp)
RVQ_SRCS=(src/legacy_rvq/gas_legacy/anns/RVQ/RVQ.cu src/legacy_rvq/gas_legacy/anns/functions/distance_kernel.cu
          src/legacy_rvq/gas_legacy/anns/functions/selectMin1.cu src/search/rvq_entry_provider.cpp
          src/search/rvq_device_entries.cu)
OBJS=()
for s in "${SRCS[@]}"; do
    o="$OUT/obj/$(basename "${s%.*}").o"
    OBJS+=("$o")
    if [[ ! -f "$o" || "$REF/$s" -nt "$o" ]]; then
        echo "[ref_build] $s"
        "$NVCC" "${FLAGS[@]}" -x cu -c "$REF/$s" -o "$o"
    fi
done
for s in "${RVQ_SRCS[@]}"; do
    o="$OUT/obj/$(basename "${s%.*}").o"
    OBJS+=("$o")
    if [[ ! -f "$o" || "$REF/$s" -nt "$o" ]]; then
        echo "[ref_build] $s"
        "$NVCC" "${FLAGS[@]}" "${RVQ_FLAGS[@]}" -x cu -c "$REF/$s" -o "$o"
    fi
done
"$NVCC" "${FLAGS[@]}" -x cu -c "$HERE/ref_stub.cu" -o "$OUT/obj/ref_stub.o"
"$NVCC" "${FLAGS[@]}" "${RVQ_FLAGS[@]}" -x cu -c "$HERE/ref_shim/cblas_shim.cpp" -o "$OUT/obj/cblas_shim.o"
"$NVCC" "${FLAGS[@]}" -x cu -c "$HERE/ref_driver.cpp" -o "$OUT/obj/ref_driver.o"
"$NVCC" -gencode arch=compute_100a,code=sm_100a -rdc=true -o "$OUT/ref_driver" "${OBJS[@]}" \
    "$OUT/obj/ref_stub.o" "$OUT/obj/cblas_shim.o" "$OUT/obj/ref_driver.o" -lcublas
echo "[ref_build] built $OUT/ref_driver"
