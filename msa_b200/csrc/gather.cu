// Fetch of the selected documents' pooled K/V from the pinned host bank.
//
// The host bank keeps a document's chunks contiguous ([chunk][K|V][Hkv][D]), so one
// selected document is one linear run of host memory.  The gather kernel reads it through
// the device-visible mapping with 16-byte loads (PCIe reads, no staging copy, no host
// thread involved) and scatters it into the head-major [Hkv, entries, D] layout the
// attention path consumes.  Bound by PCIe bandwidth: 2*chunks*Hkv*D*e bytes per document.
#include <cstdlib>

#include "common.cuh"

namespace msa {

constexpr int kPlanThreads = 256;
constexpr int kPlanMaxK = 64;

// status[2] counts winners that were dropped because their owner rank or local id does not exist in the
// directory (a corrupt candidate, or a directory that no longer matches the bank): nothing is read for them.
__global__ void __launch_bounds__(kPlanThreads)
gather_plan_kernel(const int64_t* __restrict__ sel_local, const int32_t* __restrict__ sel_rank, int n_seq, int k,
                   int world, const int64_t* __restrict__ shard_doc_base, long long n_dir_rows,
                   const int64_t* __restrict__ doc_chunk_offset, const int32_t* __restrict__ doc_chunk_len,
                   const uint64_t* __restrict__ shard_kv_base, long long chunk_bytes, long long sample_stride,
                   int64_t* __restrict__ plan, int64_t* __restrict__ n_sel, int64_t* __restrict__ total,
                   int64_t* total_host, int32_t* __restrict__ status, int64_t* __restrict__ resident, int slot_len) {
  __shared__ long long s_scan[kPlanThreads];
  __shared__ long long s_carry;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (int base = 0; base < n_seq; base += kPlanThreads) {
    const int b = base + threadIdx.x;
    long long mine = 0;
    if (b < n_seq) {
      // insertion sort of the sample's valid winners by (owner rank, local id)
      long long key[kPlanMaxK];
      int n = 0, dropped = 0;
      for (int j = 0; j < k; ++j) {
        const long long lid = sel_local[(long long)b * k + j];
        const int r = sel_rank ? sel_rank[(long long)b * k + j] : 0;
        if (lid <= 0) continue;                            // dummy document or invalidated winner
        if (r < 0 || r >= world) { ++dropped; continue; }
        // shard r owns directory rows [base[r], base[r+1]); row base[r] is its dummy document
        const long long lo = shard_doc_base[r], hi = r + 1 < world ? shard_doc_base[r + 1] : n_dir_rows;
        if (lid >= hi - lo) { ++dropped; continue; }
        const long long kk = ((long long)r << 40) | lid;
        int p = n++;
        while (p > 0 && key[p - 1] > kk) { key[p] = key[p - 1]; --p; }
        key[p] = kk;
      }
      if (dropped && status) atomicAdd(status + 2, dropped);
      // Resident set (a decode loop that refreshes the same segment every step): the sample's room is k slots of
      // slot_len entries, resident[b][s] is the document whose entries slot s holds.  When the k winners are all
      // valid and every one holds exactly slot_len entries, the winners that are already in a slot stay where they
      // are and only the others are planned, into the slots of the documents that dropped out.  Any other sample
      // is planned in full (below) and its table is cleared.
      bool keep_slots = resident != nullptr && n == k && sample_stride == (long long)k * slot_len;
      if (keep_slots)
        for (int j = 0; j < k && keep_slots; ++j) {
          const long long d = shard_doc_base[(int)(key[j] >> 40)] + (key[j] & ((1ll << 40) - 1));
          keep_slots = doc_chunk_len[d] == slot_len;
        }
      if (keep_slots) {
        int64_t* res = resident + (long long)b * k;
        unsigned long long kept = 0ull, hit = 0ull;       // slots that keep their document; winners that have a slot
        for (int s = 0; s < k; ++s) {
          const long long have = res[s];
          for (int j = 0; j < k; ++j)
            if (have == key[j]) { kept |= 1ull << s; hit |= 1ull << j; break; }
        }
        int s = 0;
        for (int j = 0; j < k; ++j) {
          int64_t* row = plan + ((long long)b * k + j) * 4;
          row[3] = b;
          if ((hit >> j) & 1ull) { row[0] = 0; row[1] = 0; row[2] = 0; continue; }
          while ((kept >> s) & 1ull) ++s;
          kept |= 1ull << s;
          res[s] = key[j];
          const int r = (int)(key[j] >> 40);
          const long long d = shard_doc_base[r] + (key[j] & ((1ll << 40) - 1));
          row[0] = (int64_t)(shard_kv_base[r] + (unsigned long long)(doc_chunk_offset[d] * chunk_bytes));
          row[1] = slot_len;
          row[2] = (long long)s * slot_len;
        }
        mine = (long long)k * slot_len;
        n_sel[b] = mine;
      } else {
      if (resident != nullptr)
        for (int s = 0; s < k; ++s) resident[(long long)b * k + s] = -1;
      for (int j = 0; j < k; ++j) {
        int64_t* row = plan + ((long long)b * k + j) * 4;
        long long len = 0;
        if (j < n) {
          const int r = (int)(key[j] >> 40);
          const long long lid = key[j] & ((1ll << 40) - 1);
          const long long d = shard_doc_base[r] + lid;
          len = doc_chunk_len[d];
          if (sample_stride > 0 && mine + len > sample_stride) len = sample_stride - mine;   // the sample's room is full
          row[0] = (int64_t)(shard_kv_base[r] + (unsigned long long)(doc_chunk_offset[d] * chunk_bytes));
        } else {
          row[0] = 0;
        }
        row[1] = len > 0 ? len : 0;
        row[2] = len > 0 ? mine : 0;   // offset inside the sample; packed mode adds the sample's base below
        row[3] = b;
        if (len > 0) mine += len;
      }
      n_sel[b] = mine;
      }
    }
    // exclusive scan of the per-sample totals across the CTA, carried between rounds
    s_scan[threadIdx.x] = mine;
    __syncthreads();
    for (int d = 1; d < kPlanThreads; d <<= 1) {
      const long long other = threadIdx.x >= d ? s_scan[threadIdx.x - d] : 0;
      __syncthreads();
      s_scan[threadIdx.x] += other;
      __syncthreads();
    }
    const long long excl = s_carry + s_scan[threadIdx.x] - mine;
    if (b < n_seq && sample_stride == 0)
      for (int j = 0; j < k; ++j) {
        int64_t* row = plan + ((long long)b * k + j) * 4;
        if (row[1] > 0) row[2] += excl;
      }
    __syncthreads();
    if (threadIdx.x == kPlanThreads - 1) s_carry += s_scan[kPlanThreads - 1];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    total[0] = s_carry;
    if (total_host) *reinterpret_cast<volatile int64_t*>(total_host) = s_carry;
  }
}

constexpr int kGatherThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kGatherThreads)
gather_kernel(const int64_t* __restrict__ plan, int n_items, int n_kv_heads, int head_dim, T* __restrict__ out_k,
              T* __restrict__ out_v, long long out_head_stride, long long out_entries, long long out_sample_stride) {
  constexpr int V = Elem<T>::kVec;
  const int vec_half = n_kv_heads * head_dim / V;  // 16-byte vectors in one chunk's K (or V)
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
  const int64_t* row = plan + (long long)item * 4;
  const long long dst0 = row[2];
  // clamp once: nothing is read for entries that have no room (out_entries counts per sample when the
  // destination is strided by sample, over the whole output otherwise)
  const long long len = min((long long)row[1], out_entries - dst0);
  if (len <= 0) continue;
  const uint4* src = reinterpret_cast<const uint4*>((uintptr_t)row[0]);
  const long long sample_off = out_sample_stride * row[3];
  const long long n_vec = len * 2 * vec_half;
  // each thread keeps four independent 16-byte PCIe reads in flight
  for (long long v0 = threadIdx.x; v0 < n_vec; v0 += 4ll * kGatherThreads) {
    uint4 val[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long v = v0 + (long long)u * kGatherThreads;
      if (v < n_vec) val[u] = src[v];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long v = v0 + (long long)u * kGatherThreads;
      if (v >= n_vec) continue;
      const long long chunk = v / (2 * vec_half);
      const int w = (int)(v % (2 * vec_half));
      const int in_half = w % vec_half;
      const int h = (in_half * V) / head_dim, d = (in_half * V) % head_dim;
      const long long entry = dst0 + chunk;
      T* dst = (w < vec_half ? out_k : out_v) + sample_off + (long long)h * out_head_stride + entry * head_dim + d;
      *reinterpret_cast<uint4*>(dst) = val[u];
    }
  }
  }
}

}  // namespace msa

using namespace msa;

// The plan and gather kernels run on a side stream beside kernels that need almost all of an SM's shared memory
// (the persistent routing kernels).  A kernel with little shared memory of its own leaves the SM configured for a
// large L1, and a CTA that needs 200 KB cannot join it there until the SM has drained: measured on B200, a 3.2 GB
// routing launch took 758 us instead of 461 us next to a 24-CTA gather, because the routing CTAs of the occupied
// SMs started only when the first wave had ended.  Asking for the largest shared-memory carve-out keeps those SMs
// open (507 us).
static int prefer_shared_carveout() {
  static bool done[kMaxDevices] = {};
  int device = 0;
  MSA_OK_OR_RETURN(current_device(&device));
  if (done[device] || getenv("MSA_B200_GATHER_DEFAULT_CARVEOUT")) return MSA_OK;
  MSA_CUDA_OK(cudaFuncSetAttribute(gather_kernel<__nv_bfloat16>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   cudaSharedmemCarveoutMaxShared));
  MSA_CUDA_OK(cudaFuncSetAttribute(gather_kernel<float>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   cudaSharedmemCarveoutMaxShared));
  MSA_CUDA_OK(cudaFuncSetAttribute(gather_plan_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   cudaSharedmemCarveoutMaxShared));
  done[device] = true;
  return MSA_OK;
}

namespace {
int gather_plan_launch(const int64_t* sel_local, const int32_t* sel_rank, int32_t n_seq, int32_t k, int32_t world,
                       const int64_t* shard_doc_base, int64_t n_dir_rows, const int64_t* doc_chunk_offset,
                       const int32_t* doc_chunk_len, const uint64_t* shard_kv_base, int64_t chunk_bytes,
                       int64_t sample_stride, int64_t* plan, int64_t* n_sel, int64_t* total, int64_t* total_host_mapped,
                       int32_t* status, int64_t* resident, int32_t slot_len, void* stream) {
  MSA_REQUIRE(sel_local && shard_doc_base && doc_chunk_offset && doc_chunk_len && shard_kv_base && plan && n_sel &&
                  total, "gather_plan: null pointer");
  MSA_REQUIRE(n_seq >= 0 && k >= 1 && k <= kPlanMaxK && world >= 1, "gather_plan: bad sizes (k must be <= %d)",
              kPlanMaxK);
  MSA_REQUIRE(n_dir_rows >= world, "gather_plan: n_dir_rows=%lld is smaller than the %d dummy rows of the shards",
              (long long)n_dir_rows, world);
  MSA_REQUIRE(chunk_bytes > 0 && chunk_bytes % 16 == 0, "gather_plan: chunk_bytes must be a multiple of 16");
  MSA_REQUIRE(sample_stride >= 0, "gather_plan: sample_stride must not be negative");
  MSA_REQUIRE(resident == nullptr || (slot_len > 0 && sample_stride == (int64_t)k * slot_len),
              "gather_plan: a resident table needs sample_stride == k * slot_len");
  MSA_OK_OR_RETURN(prefer_shared_carveout());
  gather_plan_kernel<<<1, kPlanThreads, 0, (cudaStream_t)stream>>>(
      sel_local, sel_rank, n_seq, k, world, shard_doc_base, n_dir_rows, doc_chunk_offset, doc_chunk_len, shard_kv_base,
      chunk_bytes, sample_stride, plan, n_sel, total, total_host_mapped, status, resident, slot_len);
  MSA_LAUNCH_OK("gather_plan_kernel");
  return MSA_OK;
}
}  // namespace

extern "C" int msa_gather_plan(const int64_t* sel_local, const int32_t* sel_rank, int32_t n_seq, int32_t k,
                               int32_t world, const int64_t* shard_doc_base, int64_t n_dir_rows,
                               const int64_t* doc_chunk_offset, const int32_t* doc_chunk_len,
                               const uint64_t* shard_kv_base, int64_t chunk_bytes, int64_t sample_stride,
                               int64_t* plan, int64_t* n_sel, int64_t* total, int64_t* total_host_mapped,
                               int32_t* status, void* stream) {
  return gather_plan_launch(sel_local, sel_rank, n_seq, k, world, shard_doc_base, n_dir_rows, doc_chunk_offset, doc_chunk_len,
                            shard_kv_base, chunk_bytes, sample_stride, plan, n_sel, total, total_host_mapped, status, nullptr,
                            0, stream);
}

extern "C" int msa_gather_plan_resident(const int64_t* sel_local, const int32_t* sel_rank, int32_t n_seq, int32_t k,
                                        int32_t world, const int64_t* shard_doc_base, int64_t n_dir_rows,
                                        const int64_t* doc_chunk_offset, const int32_t* doc_chunk_len,
                                        const uint64_t* shard_kv_base, int64_t chunk_bytes, int32_t slot_len,
                                        int64_t* resident, int64_t* plan, int64_t* n_sel, int64_t* total,
                                        int32_t* status, void* stream) {
  MSA_REQUIRE(resident != nullptr, "gather_plan_resident: null pointer");
  return gather_plan_launch(sel_local, sel_rank, n_seq, k, world, shard_doc_base, n_dir_rows, doc_chunk_offset, doc_chunk_len,
                            shard_kv_base, chunk_bytes, (int64_t)k * slot_len, plan, n_sel, total, nullptr, status, resident,
                            slot_len, stream);
}

extern "C" int msa_gather_run(const int64_t* plan, int32_t n_items, int32_t dtype, int32_t n_kv_heads,
                              int32_t head_dim, void* out_k, void* out_v, int64_t out_head_stride,
                              int64_t out_entries, int64_t out_sample_stride, int32_t max_ctas, void* stream) {
  MSA_REQUIRE(dtype_ok(dtype), "gather_run: unknown dtype %d", dtype);
  MSA_REQUIRE(plan && n_items >= 0 && n_kv_heads > 0 && head_dim > 0 && max_ctas >= 0 && out_sample_stride >= 0,
              "gather_run: bad arguments");
  // The link is saturated by a few hundred KB of reads in flight (16 KB per CTA).  Measured on B200 with
  // 32 KiB documents: 49.8 GB/s alone from 12 CTAs up; next to the HBM-bound decode-time scoring the
  // neighbour loses 0.18 ms per layer with 512 CTAs and 0.05 ms with 16-32; next to the tensor-bound prefill
  // scoring one CTA per document is best (35 GB/s against 20 GB/s at 24 CTAs).
  const int grid = (max_ctas > 0 && max_ctas < n_items) ? max_ctas : n_items;
  const int vec = 16 / (int)dtype_size(dtype);
  MSA_REQUIRE(head_dim % vec == 0 && out_head_stride % vec == 0 && out_sample_stride % vec == 0,
              "gather_run: rows must be 16-byte multiples");
  if (n_items == 0 || out_entries == 0) return MSA_OK;
  MSA_REQUIRE(out_k && out_v && aligned16(out_k) && aligned16(out_v), "gather_run: bad output pointers");
  MSA_OK_OR_RETURN(prefer_shared_carveout());
  if (dtype == MSA_BF16)
    gather_kernel<__nv_bfloat16><<<grid, kGatherThreads, 0, (cudaStream_t)stream>>>(
        plan, n_items, n_kv_heads, head_dim, (__nv_bfloat16*)out_k, (__nv_bfloat16*)out_v, out_head_stride, out_entries,
        out_sample_stride);
  else
    gather_kernel<float><<<grid, kGatherThreads, 0, (cudaStream_t)stream>>>(
        plan, n_items, n_kv_heads, head_dim, (float*)out_k, (float*)out_v, out_head_stride, out_entries,
        out_sample_stride);
  MSA_LAUNCH_OK("gather_kernel");
  return MSA_OK;
}
