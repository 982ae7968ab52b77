// Interface between the planner / C ABI of a resident program (resident_host.cu) and its
// persistent kernel (resident.cu).
#pragma once
#include "common.cuh"
#include "resident.cuh"

namespace fml {
namespace res {

struct KernelArgs {
  const Step *steps;                       // the CTAs' step lists back to back, each ended by kEnd
  const int32_t *step_begin;               // [ctas]: first step of each CTA
  const GemmStage *gemm;
  const AttnStage *attn;
  const uint8_t *weights;                  // packed weight streams
  const unsigned long long *weight_begin;  // [ctas]: byte offset of each CTA's stream
  unsigned *epoch;                         // pass number: selects the parity of every buffer generation
  unsigned *abort_word;                    // set by whichever CTA gives up a wait first
  int *status;
  unsigned long long *trace;               // traced variant only: [cta][max_steps][kTraceSlots]
  int32_t nslots, slot_bytes, overlay_bytes, max_steps;
};

size_t kernel_smem_bytes(int nslots, int slot_bytes, int overlay_bytes);
int launch_resident_kernel(const KernelArgs &args, int ctas, size_t smem_bytes, bool trace, cudaStream_t stream);

}  // namespace res
}  // namespace fml
