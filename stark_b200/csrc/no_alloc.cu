// stark_b200_op_attention_decode_static: decode attention for callers that must not allocate.
//
// Who that is: a serving worker decides up front how much device memory a request may use (the
// reference's workers refuse a request whose estimate does not fit and never grow afterwards), and
// a decode loop cannot afford cudaMalloc / cudaFree at all, because both stall every stream of the
// device.  Such a caller owns all of its buffers, including the KV pages, and only needs the
// kernel.  The kernel, however, needs working memory of its own for the split-KV partial results
// and the per-head arrival counters.  Here that memory is a fixed array that lives in the library
// image: every GPU that loads the library carries it (1 MiB) until the process exits, nothing is
// allocated per call, and the price is a hard upper bound on the problem size.
#include <cmath>
#include <cstdint>

#include "ops.cuh"

constexpr size_t kStaticScratchBytes = 1u << 20;  // the stated maximum; see static_attention_fits()
constexpr size_t kHeaderBytes = 1024;             // [0, 256): arrival counters, [256, 288): step state
constexpr size_t kStateOffset = 256;
constexpr uint32_t kMaxStaticKvHeads = 64;

// Working memory of the static entry point.  In host code this name is only a handle for
// cudaGetSymbolAddress; device code may use it directly (static_prepare_kernel does).
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on each device, resolved on the first call per device.
static void *g_scratch_address[64] = {nullptr};

namespace sb {

namespace {

// Every call starts from zeroed arrival counters and its own position; the partial results need
// no clearing because each launch overwrites every entry it later reads.
__global__ void static_prepare_kernel(uint32_t position, uint32_t kv_heads) {
    uint32_t *counters = reinterpret_cast<uint32_t *>(g_static_scratch);
    StepState *state = reinterpret_cast<StepState *>(g_static_scratch + kStateOffset);
    if (threadIdx.x < kv_heads) counters[threadIdx.x] = 0u;
    if (threadIdx.x == 0) {
        state->position = position;
        state->token = 0u;
        state->next_token = 0u;
        state->cursor = 0u;
        state->gen_cursor = 0u;
        state->gen_capacity = 0u;
    }
}

bool static_attention_fits(uint32_t q_heads, uint32_t kv_heads, uint32_t splits) {
    if (kv_heads == 0 || kv_heads > kMaxStaticKvHeads) return false;
    const size_t need = attention_scratch_floats(q_heads, kv_heads, splits) * sizeof(float);
    return need <= kStaticScratchBytes - kHeaderBytes;
}

}  // namespace

}  // namespace sb

using namespace sb;

extern "C" stark_b200_status stark_b200_op_attention_decode_static(
    const void *qkv, void *key_pages, void *value_pages, const int32_t *block_table, void *out,
    const float *q_norm, const float *k_norm, const float *rope_cos, const float *rope_sin,
    const stark_b200_attention_desc *desc, void *stream) {
    if (!qkv || !key_pages || !value_pages || !block_table || !out || !desc) return STARK_B200_INVALID_ARGUMENT;
    if (desc->struct_size != sizeof(stark_b200_attention_desc) || desc->abi_version != STARK_B200_ABI_VERSION)
        return STARK_B200_ABI_MISMATCH;
    if (desc->head_dim != kHeadDim || desc->kv_heads == 0 || desc->q_heads % desc->kv_heads != 0 ||
        desc->q_heads / desc->kv_heads > 8u)
        return STARK_B200_UNSUPPORTED;
    if ((rope_cos == nullptr) != (rope_sin == nullptr)) return STARK_B200_INVALID_ARGUMENT;
    const uint32_t splits = desc->splits ? desc->splits : 8u;
    if (splits > kMaxAttnSplits) return STARK_B200_INVALID_ARGUMENT;
    // The fixed working memory bounds the problem: q_heads * splits * 520 bytes must fit in 1 MiB - 1 KiB.
    if (!static_attention_fits(desc->q_heads, desc->kv_heads, splits)) return STARK_B200_CONTEXT_LIMIT;

    int device = 0;
    SB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return STARK_B200_UNSUPPORTED;
    if (!g_scratch_address[device]) {
        // First call on this device (the device is current here): turn the symbol into a device address.
        void *address = nullptr;
        SB_CUDA(cudaGetSymbolAddress(&address, g_static_scratch));
        if (!address) return STARK_B200_DEVICE_FAILURE;
        g_scratch_address[device] = address;
    }
    unsigned char *base = static_cast<unsigned char *>(g_scratch_address[device]);
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    static_prepare_kernel<<<1, kMaxStaticKvHeads, 0, s>>>(desc->position, desc->kv_heads);
    SB_CUDA(cudaGetLastError());

    AttnArgs a{};
    a.qkv = static_cast<const uint16_t *>(qkv);
    a.out = static_cast<uint16_t *>(out);
    a.kv = KvLayer{static_cast<uint16_t *>(key_pages), static_cast<uint16_t *>(value_pages)};
    a.block_table = block_table;
    a.q_norm = q_norm;
    a.k_norm = k_norm;
    a.rope_cos = rope_cos;
    a.rope_sin = rope_sin;
    a.state = reinterpret_cast<const StepState *>(base + kStateOffset);
    a.eps = desc->epsilon;
    a.scale = 1.0f / sqrtf((float)kHeadDim);
    a.q_heads = desc->q_heads;
    a.kv_heads = desc->kv_heads;
    a.splits = splits;
    a.scratch = reinterpret_cast<float *>(base + kHeaderBytes);
    a.counters = reinterpret_cast<uint32_t *>(base);
    a.error_word = nullptr;
    a.trace = nullptr;
    a.pdl = false;
    return attention_decode_launch(a, s);
}
