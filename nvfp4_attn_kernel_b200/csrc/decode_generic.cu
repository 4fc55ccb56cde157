// CUDA-core decode kernel.  One CTA of 128 threads per (split, KV head, row);
// handles every group size G = Hq/Hkv in {1,2,4,8,16,32}.  It follows the attention
// oracle step by step (backward page walk, exact running maximum, P quantised to
// NVFP4 per 16 kv positions with the oracle's division form, BF16 P for the tail)
// and is both the fallback for shapes the tensor-core kernel does not take and the
// on-device cross-check for it.
#include "decode_common.cuh"

namespace nvfp4 {

constexpr int kRowPad = 80;  // packed 64-byte rows padded to 80 bytes in shared memory

template <int G>
struct GenericSmem {
  __align__(16) uint8_t kp[kPage * kRowPad];
  __align__(16) uint8_t vp[kHeadDim * kRowPad];
  __align__(16) uint8_t ksf[kSfBlockBytes];
  __align__(16) uint8_t vsf[kSfBlockBytes];
  __align__(16) float qf[G * kHeadDim];  // dequantised NVFP4 query
  __align__(16) float qb[G * kHeadDim];  // BF16 query (tail)
  __align__(16) float pf[G * kHeadDim];  // P of the current block
  float red[4 * G];
};

__device__ __forceinline__ void decode16(const uint2 w, float* out) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    out[i] = e2m1_to_f32((w.x >> (4 * i)) & 15u);
    out[8 + i] = e2m1_to_f32((w.y >> (4 * i)) & 15u);
  }
}

template <int G>
__global__ void __launch_bounds__(128) decode_generic_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  GenericSmem<G>& sm = *reinterpret_cast<GenericSmem<G>*>(smem_raw);
  const int tid = threadIdx.x;
  const TileWork w = resolve_grid_work(p);

  // ---- query: dequantise the G heads of this KV head ----
  for (int it = tid; it < G * 8; it += 128) {
    const int q = it >> 3, g = it & 7;
    const int head = w.kvh * G + q;
    uint2 pk;
    float sc;
    if (p.q_fp4) {
      pk = *reinterpret_cast<const uint2*>(p.q_fp4 + ((int64_t)w.row * p.heads_q + head) * 64 + g * 8);
      sc = e4m3_to_f32(p.q_sf[(int64_t)w.row * p.heads_q * kSfBlockBytes +
                              (int64_t)w.kvh * kSfBlockBytes + sf_offset(q, g)]);
    } else {
      // no quantised query was supplied: quantise the BF16 group here (stand-alone quantiser's arithmetic)
      const uint16_t* qsrc = p.q_bf16 + (int64_t)w.row * p.q_row_stride + (int64_t)head * p.q_head_stride + g * 16;
      float x[16];
      unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(qsrc)), x);
      unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(qsrc) + 1), x + 8);
      uint8_t sf;
      quantize_group16(x, pk.x, pk.y, sf);
      sc = e4m3_to_f32(sf);
    }
    float v[16];
    decode16(pk, v);
#pragma unroll
    for (int i = 0; i < 16; ++i) sm.qf[q * kHeadDim + g * 16 + i] = v[i] * sc;
    if (w.tail_len > 0 && p.q_bf16) {
      const uint16_t* src = p.q_bf16 + (int64_t)w.row * p.q_row_stride + (int64_t)head * p.q_head_stride + g * 16;
#pragma unroll
      for (int i = 0; i < 16; ++i) sm.qb[q * kHeadDim + g * 16 + i] = bf16_bits_to_f32(src[i]);
    }
  }
  __syncthreads();

  float m[G], l[G], o[G];
#pragma unroll
  for (int q = 0; q < G; ++q) { m[q] = -INFINITY; l[q] = 0.f; o[q] = 0.f; }

  if (w.tail_len > 0) {
    // without a BF16 query the tail scores fall back to the dequantised one
    tail_block<G>(p, w, p.q_bf16 ? sm.qb : sm.qf, sm.pf, sm.red, tid, 0, m, l, o);
  }

  for (int page = w.last_page - 1; page >= w.first_page; --page) {
    const int64_t pid = p.page_table[(int64_t)w.row * p.page_table_row_stride + page];
    if (pid < 0 || pid >= p.num_pages) {
      if (tid == 0) set_status(p.status, NVFP4_STATUS_BAD_PAGE_ID);
      continue;
    }
    // ---- stage the page-head tile ----
    {
      const uint8_t* kg = p.k_packed + pid * p.k_pitch + (int64_t)w.kvh * 64;
      const uint8_t* vg = p.v_packed + pid * p.v_pitch + (int64_t)w.kvh * kHeadDim * 64;
      const int64_t krow_stride = (int64_t)p.heads_kv * 64;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = j * 32 + (tid >> 2), c = tid & 3;
        *reinterpret_cast<uint4*>(sm.kp + r * kRowPad + c * 16) =
            __ldg(reinterpret_cast<const uint4*>(kg + r * krow_stride + c * 16));
        *reinterpret_cast<uint4*>(sm.vp + r * kRowPad + c * 16) =
            __ldg(reinterpret_cast<const uint4*>(vg + r * 64 + c * 16));
      }
      if (tid < 64) {
        reinterpret_cast<uint4*>(sm.ksf)[tid] = __ldg(reinterpret_cast<const uint4*>(
            p.k_sf + pid * p.k_sf_pitch + (int64_t)w.kvh * kSfBlockBytes) + tid);
      } else {
        reinterpret_cast<uint4*>(sm.vsf)[tid - 64] = __ldg(reinterpret_cast<const uint4*>(
            p.v_sf + pid * p.v_sf_pitch + (int64_t)w.kvh * kSfBlockBytes) + (tid - 64));
      }
    }
    __syncthreads();

    // ---- scores: thread = kv position ----
    float z[G];
#pragma unroll
    for (int q = 0; q < G; ++q) z[q] = 0.f;
#pragma unroll 2
    for (int g = 0; g < 8; ++g) {
      float kv[16];
      decode16(*reinterpret_cast<const uint2*>(sm.kp + tid * kRowPad + g * 8), kv);
      const float sc = e4m3_to_f32(sm.ksf[sf_offset(tid, g)]);
#pragma unroll
      for (int q = 0; q < G; ++q) {
        const float4* qv = reinterpret_cast<const float4*>(sm.qf + q * kHeadDim + g * 16);
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 a = qv[i];
          acc = fmaf(kv[4 * i], a.x, acc); acc = fmaf(kv[4 * i + 1], a.y, acc);
          acc = fmaf(kv[4 * i + 2], a.z, acc); acc = fmaf(kv[4 * i + 3], a.w, acc);
        }
        z[q] = fmaf(sc, acc, z[q]);
      }
    }
    float bm[G], resc[G];
#pragma unroll
    for (int q = 0; q < G; ++q) { z[q] *= p.scale_log2; bm[q] = z[q]; }
    block_max_128<G>(bm, sm.red, tid, 0);
#pragma unroll
    for (int q = 0; q < G; ++q) {
      const float mn = fmaxf(m[q], bm[q]);
      resc[q] = (m[q] == -INFINITY) ? 0.f : exp2f(m[q] - mn);
      m[q] = mn;
      const float pe = exp2_rel(z[q], mn);
      l[q] = fmaf(l[q], resc[q], pe);
      // NVFP4 round trip of P over the 16 kv positions of this half-warp
      const float gmax = halfwarp_max(pe);
      const uint8_t sb = p_scale_byte(gmax);
      float pq = pe;  // a group whose scale rounds to zero passes through, as in the oracle
      if (sb != 0) {
        const float sc = e4m3_to_f32(sb);
        pq = e2m1_to_f32(f32_to_e2m1(__fdiv_rn(pe, sc))) * sc;
      }
      sm.pf[q * kHeadDim + tid] = pq;
    }
    __syncthreads();

    // ---- P.V: thread = channel ----
#pragma unroll
    for (int q = 0; q < G; ++q) o[q] *= resc[q];
#pragma unroll 2
    for (int g = 0; g < 8; ++g) {
      float vv[16];
      decode16(*reinterpret_cast<const uint2*>(sm.vp + tid * kRowPad + g * 8), vv);
      const float sc = e4m3_to_f32(sm.vsf[sf_offset(tid, g)]);
#pragma unroll
      for (int q = 0; q < G; ++q) {
        const float4* pv = reinterpret_cast<const float4*>(sm.pf + q * kHeadDim + g * 16);
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 a = pv[i];
          acc = fmaf(vv[4 * i], a.x, acc); acc = fmaf(vv[4 * i + 1], a.y, acc);
          acc = fmaf(vv[4 * i + 2], a.z, acc); acc = fmaf(vv[4 * i + 3], a.w, acc);
        }
        o[q] = fmaf(sc, acc, o[q]);
      }
    }
    __syncthreads();
  }

  write_output<G>(p, w, sm.red, tid, 0, m, l, o);
}

template <int G>
static cudaError_t launch_g(const DecodeParams& p, cudaStream_t stream) {
  const size_t smem = sizeof(GenericSmem<G>);
  static bool configured[64] = {};  // per device; the attribute belongs to the device's context
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(decode_generic_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid(p.num_splits, p.heads_kv, p.rows);
  decode_generic_kernel<G><<<grid, 128, smem, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_decode_generic(const DecodeParams& p, cudaStream_t stream) {
  if (p.rows == 0) return cudaSuccess;
  switch (p.heads_q / p.heads_kv) {
    case 1: return launch_g<1>(p, stream);
    case 2: return launch_g<2>(p, stream);
    case 3: return launch_g<3>(p, stream);
    case 4: return launch_g<4>(p, stream);
    case 5: return launch_g<5>(p, stream);
    case 6: return launch_g<6>(p, stream);
    case 7: return launch_g<7>(p, stream);
    case 8: return launch_g<8>(p, stream);
    case 16: return launch_g<16>(p, stream);
    case 32: return launch_g<32>(p, stream);
    default: return cudaErrorNotSupported;
  }
}

}  // namespace nvfp4
