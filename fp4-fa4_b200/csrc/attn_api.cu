// Host side of the attention entry points: argument checks, workspace layout.
#include "attn.cuh"

using namespace fa4b;

extern "C" {

int fa4b_query(fa4b_info* out) {
  FA4B_REQUIRE(out != nullptr, FA4B_BAD_ARG, "fa4b_query: out is NULL");
  *out = fa4b_info{};
  out->abi_version = FA4B_ABI_VERSION;
  out->build_sm = 100;
  out->tile_q = 128;
  out->tile_kv = 128;
  out->wait_limit = (int)(kWaitLimitCycles / 2000000);  // ms at 2 GHz
  fill_kernel_info(out);
  return FA4B_OK;
}

size_t fa4b_attn_workspace_bytes(const fa4b_attn_dims* d) {
  fa4b_attn_ws_layout l;
  if (fa4b_attn_ws_layout_query(d, &l) != FA4B_OK) return 0;
  return l.total;
}

int fa4b_attn_ws_layout_query(const fa4b_attn_dims* d, fa4b_attn_ws_layout* out) {
  FA4B_REQUIRE(d && out, FA4B_BAD_ARG, "NULL argument");
  if (int s = check_dims(*d)) return s;
  *out = make_ws_layout(*d);
  return FA4B_OK;
}

}  // extern "C"

extern "C" int fa4b_attn_check_status(const fa4b_attn_dims* d, const void* ws, void* stream) {
  FA4B_REQUIRE(d != nullptr, FA4B_BAD_ARG, "NULL argument");
  if (int s = check_dims(*d)) return s;
  const fa4b_attn_ws_layout l = make_ws_layout(*d);
  if (ws == nullptr) {  // the built-in cache of fa4b_attn_fwd_static on the current device
    FA4B_REQUIRE(l.saved_total <= FA4B_STATIC_WS_BYTES, FA4B_BAD_SHAPE, "ws is NULL and this shape does not fit the built-in operand cache");
    void* p = nullptr;
    if (int s = static_ws_pointer(&p)) return s;
    ws = p;
  }
  uint32_t host[4] = {0, 0, 0, 0};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FA4B_CUDA(cudaMemcpyAsync(host, static_cast<const uint8_t*>(ws) + l.status, sizeof(host), cudaMemcpyDeviceToHost, st));
  FA4B_CUDA(cudaStreamSynchronize(st));
  FA4B_REQUIRE(host[0] == 0, FA4B_TIMEOUT, "a device-side wait ran out (site %u, block %u, detail %u)", host[1], host[2], host[3]);
  return FA4B_OK;
}

extern "C" int fa4b_attn_bwd(const fa4b_attn_bwd_args* a, void* stream) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  return launch_attn_bwd(*a, static_cast<cudaStream_t>(stream));
}

extern "C" int fa4b_attn_merge(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part, int64_t n_rows, int32_t D,
                               void* o_out, void* stream) {
  return launch_attn_merge(o_acc, lse_acc, o_part, lse_part, n_rows, D, o_out, static_cast<cudaStream_t>(stream));
}

extern "C" int fa4b_attn_accumulate(float* acc, const void* part, int64_t n, void* out, void* stream) {
  return launch_attn_accumulate(acc, part, n, out, static_cast<cudaStream_t>(stream));
}
