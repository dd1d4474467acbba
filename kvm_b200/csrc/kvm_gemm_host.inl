// Host planning of the tensor-core tasks: for every matmul_mma_bf16 task whose operands TMA can address (bf16 storage,
// 16-byte aligned base, row stride a multiple of 16 bytes, tile origin on an 8-element boundary) encode the two tensor maps
// (deduplicated per GEMM) and mark the task for the tcgen05 path; everything else keeps the SIMT path.
#include <map>
#include <tuple>
#include <vector>

typedef CUresult (*KvmEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static KvmEncodeTiled kvm_encode_fn() {
  static KvmEncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (KvmEncodeTiled)p;
  }
  return fn;
}

// 2-D bf16 map over a row-major region: `inner` contiguous elements per row, `outer` rows, row stride ld elements.
static int kvm_tmap_bf16(KvmExec* h, std::map<std::tuple<void*, int, int, int, int, int>, int>& cache, void* base, int inner, int outer, int ld, int box_inner, int box_outer) {
  auto key = std::make_tuple(base, inner, outer, ld, box_inner, box_outer);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  KvmEncodeTiled enc = kvm_encode_fn();
  if (!enc) return -1;
  CUtensorMap m;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -1;
  h->tmaps.push_back(m);
  const int idx = (int)h->tmaps.size() - 1;
  cache[key] = idx;
  return idx;
}

static int kvm_plan_tc(KvmExec* h, int first_task) {
  if (h->cfg.flags & KVM_CFG_NO_TENSOR_CORES) return 0;
  std::map<std::tuple<void*, int, int, int, int, int>, int> cache;
  for (size_t i = first_task; i < h->tasks.size(); ++i) {
    const KvmTaskDesc& d = h->tasks[i];
    if (d.op_id == 45 || d.op_id == 47 || d.op_id == 48) {
      // tensor-core attention: bf16 q / k / v (/ dO), head dimension 64, whole 128-row blocks, TMA-addressable rows
      const int32_t* a = h->args.data() + d.args_off;
      const bool fwd = d.op_id == 45, dkv = d.op_id == 48;
      const int nb = fwd ? 5 : dkv ? 8 : 7;                       // buffer argument count
      const int b = a[nb], hh = a[nb + 1], r0 = a[nb + 2], T = a[nb + 3], H = a[nb + 4];
      const int hd = dkv ? a[nb + 5] : a[nb + 6];
      const KvmBuf& Q = h->bufs[a[0]]; const KvmBuf& K = h->bufs[a[1]]; const KvmBuf& V = h->bufs[a[2]];
      const KvmBuf* DO = fwd ? nullptr : &h->bufs[a[3]];
      if (hd != 64 || T <= 0 || (T & 127) || (r0 & 127) || r0 < 0 || r0 >= T || b < 0 || H <= 0 || (K.cols % 64)) continue;
      const int Hkv = dkv ? K.cols / 64 : a[nb + 5];
      if (Hkv <= 0 || H % Hkv || hh < 0 || hh >= (dkv ? Hkv : H)) continue;
      const long long R = (long long)(b + 1) * T;
      bool okb = true;
      for (const KvmBuf* B : {&Q, &K, &V, DO}) if (B && (B->dtype != KVM_BF16 || (B->ld & 7) || ((uintptr_t)B->p & 15) || B->rows < R)) okb = false;
      if (!okb || Q.cols < H * 64 || K.cols < Hkv * 64 || V.cols < Hkv * 64 || (DO && DO->cols < H * 64)) continue;
      // outputs and the lse / delta vectors are checked here too: the tensor-core bodies assume a valid geometry
      bool oko = true;
      auto mat = [&](int idx, int cols) { const KvmBuf& B = h->bufs[idx]; if (B.dtype == KVM_I32 || B.rows < R || B.cols < cols) oko = false; };
      auto vec = [&](int idx) { const KvmBuf& B = h->bufs[idx]; if (B.dtype != KVM_F32 || B.ld != B.cols || (long long)B.rows * B.cols < R * H) oko = false; };
      if (fwd) { mat(a[3], H * 64); vec(a[4]); }
      else if (!dkv) { vec(a[4]); vec(a[5]); mat(a[6], H * 64); }
      else { vec(a[4]); vec(a[5]); mat(a[6], Hkv * 64); mat(a[7], Hkv * 64); }
      if (!oko) continue;
      const int tq = kvm_tmap_bf16(h, cache, Q.p, Q.cols, Q.rows, Q.ld, 64, 128), tk = kvm_tmap_bf16(h, cache, K.p, K.cols, K.rows, K.ld, 64, 128),
                tv = kvm_tmap_bf16(h, cache, V.p, V.cols, V.rows, V.ld, 64, 128), tdo = DO ? kvm_tmap_bf16(h, cache, DO->p, DO->cols, DO->rows, DO->ld, 64, 128) : 0;
      if (tq < 0 || tk < 0 || tv < 0 || tdo < 0) continue;
      h->aux[i] = make_int4(2 | (tdo << 8), tq, tk, tv);
      continue;
    }
    if (d.op_id != 122) continue;
    const int32_t* a = h->args.data() + d.args_off;
    const KvmBuf& A = h->bufs[a[0]];
    const KvmBuf& B = h->bufs[a[1]];
    const int m0 = a[6], n0 = a[7], M = a[8], N = a[9], K = a[10], fl = a[11];
    const bool ta = fl & 1, tb = fl & 2;
    if (A.dtype != KVM_BF16 || B.dtype != KVM_BF16 || (A.ld & 7) || (B.ld & 7) || ((uintptr_t)A.p & 15) || ((uintptr_t)B.p & 15) || (m0 & 7) || (n0 & 7) || M <= 0 || N <= 0 || K <= 0)
      continue;
    if ((ta ? (A.rows < K || A.cols < M) : (A.rows < M || A.cols < K)) || (tb ? (B.rows < N || B.cols < K) : (B.rows < K || B.cols < N))) continue;   // the op reports it
    const int ia = ta ? kvm_tmap_bf16(h, cache, A.p, M, K, A.ld, 64, 64) : kvm_tmap_bf16(h, cache, A.p, K, M, A.ld, 64, 128);
    const int ib = tb ? kvm_tmap_bf16(h, cache, B.p, K, N, B.ld, 64, 256) : kvm_tmap_bf16(h, cache, B.p, N, K, B.ld, 64, 64);
    if (ia < 0 || ib < 0) continue;
    h->aux[i] = make_int4(1, ia, ib, 0);
  }
  // Partner tiles: two tensor-core tiles of the same product whose rows start at m0 (a multiple of 256) and m0 + 128 and that
  // wait for no version; each records the other (index + 1) in word 3 of its path selector, the workers may then run them
  // stacked as one 256 x 256 tile.
  if (kvm_feature_on("KVM_B200_PAIRING", (h->cfg.flags & KVM_CFG_PAIR_TILES) ? 1 : 0)) {
    std::map<std::vector<int32_t>, int> even;
    auto key_of = [&](size_t i, int m0) {
      const int32_t* a = h->args.data() + h->tasks[i].args_off;
      std::vector<int32_t> k(a, a + 13);
      k[6] = m0;
      return k;
    };
    for (size_t i = first_task; i < h->tasks.size(); ++i) {
      const KvmTaskDesc& d = h->tasks[i];
      if (d.op_id != 122 || h->aux[i].x != 1 || d.wait_var >= 0 || d.args_words < 13) continue;
      const int m0 = (h->args.data() + d.args_off)[6];
      if ((m0 & 255) == 0) even[key_of(i, m0)] = (int)i;
    }
    for (size_t i = first_task; i < h->tasks.size(); ++i) {
      const KvmTaskDesc& d = h->tasks[i];
      if (d.op_id != 122 || h->aux[i].x != 1 || d.wait_var >= 0 || d.args_words < 13) continue;
      const int32_t* a = h->args.data() + d.args_off;
      if ((a[6] & 255) != 128) continue;
      auto it = even.find(key_of(i, a[6] - 128));
      if (it == even.end() || h->aux[it->second].w != 0) continue;
      h->aux[i].w = it->second + 1;
      h->aux[it->second].w = (int)i + 1;
    }
  }
  return 0;
}
