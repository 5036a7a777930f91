// Next-token cross-entropy over materialised logits (validation mode and the
// op-level fallback for shapes the fused tensor-core head does not take).
// Per valid row: ce = max + ln(sum exp(l - max)) - l[target]
// (reference src/model.rs:3219-3227); a row is valid iff it is not the last
// step of its sequence and its target labels[row+1] != ignore_id
// (src/model.rs:27-39).
#include "kernels.hpp"

namespace ullis {
namespace k {

namespace {

__device__ __forceinline__ bool ce_row_valid(size_t row, size_t total_rows, size_t time, const uint32_t* labels,
                                             uint32_t ignore_id) {
    if (time == 0 || row % time + 1 >= time) return false;
    return row + 1 < total_rows && labels[row + 1] != ignore_id;
}

// one warp per row
__global__ void __launch_bounds__(256)
ce_rows_kernel(const float* __restrict__ logits, const uint32_t* __restrict__ labels, uint32_t ignore_id,
               size_t row0, size_t rows, size_t total_rows, size_t time, size_t vocab, float* __restrict__ row_loss,
               uint32_t* status) {
    const int lane = threadIdx.x & 31;
    const size_t local = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (local >= rows) return;
    const size_t row = row0 + local;
    if (!ce_row_valid(row, total_rows, time, labels, ignore_id)) {
        if (lane == 0) row_loss[row] = 0.0f;
        return;
    }
    const uint32_t target = labels[row + 1];
    if (target >= vocab) {
        if (lane == 0) {
            if (atomicCAS(status, ULLIS_DEV_OK, ULLIS_DEV_BAD_TOKEN) == ULLIS_DEV_OK) status[1] = (uint32_t)row;
            row_loss[row] = 0.0f;
        }
        return;
    }
    const float* l = logits + local * vocab;
    float mx = -INFINITY;
    for (size_t v = lane; v < vocab; v += 32) mx = fmaxf(mx, l[v]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
    for (size_t v = lane; v < vocab; v += 32) sum += expf(l[v] - mx);
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) row_loss[row] = mx + logf(sum) - l[target];
}

// single CTA, fixed summation tree: deterministic for a given shape
__global__ void __launch_bounds__(1024)
ce_reduce_kernel(const float* __restrict__ row_loss, const uint32_t* __restrict__ labels, uint32_t ignore_id,
                 size_t rows, size_t time, double* __restrict__ loss_sum, unsigned long long* __restrict__ n_valid,
                 double* __restrict__ pair) {
    __shared__ double s_sum[1024];
    __shared__ unsigned long long s_cnt[1024];
    double acc = 0.0;
    unsigned long long cnt = 0;
    for (size_t r = threadIdx.x; r < rows; r += 1024) {
        if (ce_row_valid(r, rows, time, labels, ignore_id)) {
            acc += (double)row_loss[r];
            cnt += 1;
        }
    }
    s_sum[threadIdx.x] = acc;
    s_cnt[threadIdx.x] = cnt;
    __syncthreads();
    for (int o = 512; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) {
            s_sum[threadIdx.x] += s_sum[threadIdx.x + o];
            s_cnt[threadIdx.x] += s_cnt[threadIdx.x + o];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        *loss_sum = s_sum[0];
        *n_valid = s_cnt[0];
        if (pair) {   // the same two numbers as doubles: the operand of the data-parallel all-reduce
            pair[0] = s_sum[0];
            pair[1] = (double)s_cnt[0];
        }
    }
}

}  // namespace

void ce_rows_from_logits(ullis_cuda_runtime* rt, const float* logits, const uint32_t* labels, uint32_t ignore_id,
                         size_t row0, size_t rows, size_t total_rows, size_t time, size_t vocab, float* row_loss) {
    if (rows == 0) return;
    ce_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, rt->stream>>>(logits, labels, ignore_id, row0, rows,
                                                                        total_rows, time, vocab, row_loss,
                                                                        rt->dev_status);
    rt->launched("ce_rows");
}

void ce_reduce(ullis_cuda_runtime* rt, const float* row_loss, const uint32_t* labels, uint32_t ignore_id,
               size_t rows, size_t time, double* loss_sum, unsigned long long* n_valid, double* pair) {
    ce_reduce_kernel<<<1, 1024, 0, rt->stream>>>(row_loss, labels, ignore_id, rows, time, loss_sum, n_valid, pair);
    rt->launched("ce_reduce");
}

}  // namespace k
}  // namespace ullis
