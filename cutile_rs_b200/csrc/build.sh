#!/usr/bin/env bash
# Builds libb200tile.so (sm_100a machine code only) next to this script's package.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
# B200_VARIANT=name builds a second library (libb200tile_name.so, objects _x.name.o) next to the
# product one:
#   B200_VARIANT=waittest B200_NVCC_EXTRA="-DB200TILE_TEST_HOOKS -DB200_WAIT_LIMIT_CYCLES=(1ll<<20)"
#       the library tests/test_wait_timeout_gpu.py loads: bounded waits give up after about half a
#       millisecond and a producer hook can leave one stage unloaded (built by __graft_entry__.build())
#   B200_VARIANT=trace B200_NVCC_EXTRA=-DB200TILE_TRACE
#       diagnostic build with cycle counters in the MMA / softmax loops and b200tile_trace_read
# The product library contains neither the hooks nor the counters.
variant="${B200_VARIANT:-}"
out="${here}/../libb200tile${variant:+_${variant}}.so"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
FLAGS=(-std=c++17 -O3 -lineinfo -gencode arch=compute_100a,code=sm_100a
       -Xcompiler -fPIC -Xcompiler -fvisibility=hidden ${B200_NVCC_EXTRA:-})
objs=()
for src in host_common gemm_tc gemm_tc_pair gemm_f32 gemm_fp8_blk gemm_nvfp4 gemm_nvfp4_pair fmha_fwd fmha_fwd_alt fmha_f32 fmha_decode gemm_host gemm_grouped norms positional argmax pointwise abi; do
  obj="${here}/_${src}${variant:+.${variant}}.o"
  if [[ ! -f "${obj}" || "${here}/${src}.cu" -nt "${obj}" || "${here}/sm100_ptx.cuh" -nt "${obj}" \
        || "${here}/host_common.h" -nt "${obj}" || "${here}/fmha_common.cuh" -nt "${obj}" || "${here}/trace.cuh" -nt "${obj}" || "${here}/../../include/b200tile.h" -nt "${obj}" ]]; then
    "${NVCC}" "${FLAGS[@]}" -c "${here}/${src}.cu" -o "${obj}" &
  fi
  objs+=("${obj}")
done
wait
"${NVCC}" -shared -o "${out}" "${objs[@]}" -lcuda 2>/dev/null || "${NVCC}" -shared -o "${out}" "${objs[@]}"
echo "built ${out}"
