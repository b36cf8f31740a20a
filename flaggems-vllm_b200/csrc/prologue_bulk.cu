// placeholder until the bulk variant lands
#include "dsv4_common.cuh"
namespace dsv4 {
cudaError_t launch_prologue_bulk(const PrologueParams& p, cudaStream_t stream) { return launch_prologue_rows(p, false, stream); }
}
