// Explicit instantiations of the grouped-GEMM launcher: __half, 1 CTA(s) per work item.  (The variants are spread
// over several translation units only so that they compile in parallel.)
#define MOE_GEMM_DEFINE_LAUNCH
#include "gemm_kernel.cuh"

namespace moe {
#define MOE_INST(BN, A_K, B_K, EPI, KG) \
  template int launch<__half, BN, A_K, B_K, EPI, KG, 1, false>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, \
                                                        const CUtensorMap&, GemmArgs, const LaunchParams&);
#define MOE_INST_BN(BN)                        \
  MOE_INST(BN, true, false, EPI_ACT, false)     \
  MOE_INST(BN, true, false, EPI_GLU, false)     \
  MOE_INST(BN, true, false, EPI_ACT_AUX, false) \
  MOE_INST(BN, true, true, EPI_ACT, false)      \
  MOE_INST(BN, true, true, EPI_ACT_AUX, false)  \
  MOE_INST(BN, true, true, EPI_DGLU, false)     \
  MOE_INST(BN, false, false, EPI_ACT, true)
MOE_INST_BN(128)
MOE_INST_BN(256)
}  // namespace moe
