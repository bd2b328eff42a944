// Placeholder translation unit for the tcgen05 backward; replaced below.
#include "common.h"
namespace ttk {
bool attn_bwd_sm100_supported(const AttnArgs&) { return false; }
size_t attn_bwd_sm100_workspace(const AttnArgs&) { return 0; }
cudaError_t attn_bwd_sm100(const AttnArgs&, void*, cudaStream_t) { return cudaErrorNotSupported; }
}  // namespace ttk
