// Decode matrix products (1..8 activation rows) for Q4_K, Q6_K and Q8_0 on the
// integer tensor cores: the streaming kernel behind llr_matmul*/llr_gemm_resident
// (one product per launch) and llr_program_run (a whole list per launch).
//
// What it computes: gemv_<t>_f32 / gemm_<t>_f32 of langtax/src/quant.rs (:6214,
// :6891, :7199 and the gemm twins), y[t][r] = sum_c W[r,c] x[t][c] with W the
// packed GGUF blocks, never expanded.  The arithmetic (activations split into
// four int8 digits, exact mma.sync dot products, integer scale folding) is
// described in llr_mma_common.cuh.
//
// Pipeline.  A CTA has ten warps with three roles and no CTA-wide barrier in
// its steady state:
//   * producer warp: walks the CTA's chunk list (16 rows x one column piece)
//     and keeps NST TMA copies in flight; a stage is refilled as soon as the eight
//     consumer warps have released it (mbarrier `empty`), not at a barrier;
//   * eight consumer warps: wait for a stage (`full`), turn their share of its
//     columns into A fragments and MMAs, release the stage, and at the end of a
//     tile hand their partial sums to a reduction buffer (`rfull`);
//   * reducer warp: adds the eight partials in warp order and writes y, so
//     results are bit-reproducible; four buffers decouple it from the math.
// Every wait is bounded; a wait that runs out sets the executor's error word
// and the warp carries on so that the kernel always terminates.
//
// One product per launch: launched with programmatic stream serialization; the
// producer prefetches before griddepcontrol.wait because weights never depend
// on earlier kernels, everything that touches activations or results waits.
//
// Program: one cooperative launch runs a list of products grouped in phases
// (independent products share a phase, e.g. attn_q|k|v).  The producer runs ahead
// across product and phase boundaries, so the next weights stream in while the
// CTA waits for its input.  A result that a later entry reads travels as tagged
// pairs {f32 bits, tag of run and phase}: the reducer stores each finished value
// with its tag, the consumers' activation split loads the pairs and spins
// (bounded) until the tags are the expected ones.  The value is its own arrival
// signal: no counter, no fence, no poll between two phases.  The split can apply
// the element-wise step that stands between two products in the model (RMSNorm,
// SwiGLU), and the reducer can add a residual vector, so a chain of products needs
// no other kernel.  Inputs that are not results of the program are plain f32; a
// program created with strict phases makes a phase with such an input wait for a
// per-phase counter (release add by every reducer, acquire polling), as a barrier.
//
// Row-sharded program (one process per GPU, each with a row slice of every matrix):
// the exchange of result slices is part of the kernel.  The reducer stores each
// finished value (plain and tagged) into its own buffers and into the same place of
// every peer's (peer stores over NVLink); consumers spin on their own GPU's copy.
// No collective library call, plain 4- and 8-byte stores only, every wait bounded.
#include <cuda_runtime.h>

#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "llr_kernels.cuh"
#include "llr_mma_common.cuh"
#include "llr_tmap.cuh"

#define LLR_ARENA_HEADER_BYTES_INTERNAL 65536  // LLR_ARENA_HEADER_BYTES of the public header


namespace llr {
namespace {
using namespace mma;

constexpr int CW = NWARP;                 // consumer warps
constexpr int NTHREADS = (CW + 2) * 32;   // + producer + reducer
constexpr int NRB = 4;                    // reduction buffers
constexpr int PART_COLS = 4096;           // columns between two hand-offs of partial sums to the reducer
constexpr int MAX_CHUNK = Lay<DT_Q4_K, 1>::CHUNK;
static_assert(Lay<DT_Q6_K, 1>::CHUNK <= MAX_CHUNK, "ring stage");
// Sharded programs keep two counter arrays in the arena header: [0, 4096) this rank's CTAs per
// phase, [4096, 8192) arrivals of the peers per phase.
constexpr int PEER_COUNTER_OFFSET = 4096;
constexpr int COUNTER_WORDS = 8192;

template <int MT> struct SLay {
  static constexpr int NT = (MT + 1) / 2;
  static constexpr int RING = 0;
  static constexpr int DIG = RING + NST * MAX_CHUNK;
  static constexpr int SXF = DIG + Sp<MT>::PLANES * Sp<MT>::DS;
  static constexpr int XSI = SXF + MT * (Sp<MT>::SPAN / 32) * 4;
  static constexpr int RED = XSI + MT * (Sp<MT>::SPAN / 256) * 4;          // float [NRB][CW][16][MT]
  static constexpr int BAR = RED + NRB * CW * 16 * MT * 4;          // full[NST] empty[NST] rfull[NRB] rempty[NRB]
  static constexpr int TOTAL = BAR + (2 * NST + 2 * NRB) * 8 + 16;
};

// How a stage of 16 rows x kseg columns reaches shared memory.
//   Q4_K, Q5_K, Q8_0, Q4_0, Q4_1, Q5_0, Q5_1: one 3-D TMA box over (words of a 256-column group, rows, groups of
//         the row): the stage is laid out [group][row][pitch].  A group is one K-quant block or eight 32-column
//         blocks; its bytes are a multiple of 16, which a box needs.  The pitch is the group's size, except
//         where that would put the fragment reads of eight rows on the same banks (Q4_1: 160 bytes, Q5_1: 192):
//         there the box is 16 bytes wider than the tensor's inner extent, and the copy engine fills the rest
//         with zeros without reading anything.  With the row order of q4k_row() the pitches 144, 176 and 208
//         spread the 4- and 8-byte fragment reads of a warp over all banks;
//   Q6_K: one 2-D box over (8-byte words of the row, rows): rows 1680 bytes apart (16 mod 128).
// One instruction per stage matters: the TMA unit of an SM accepts a bulk copy every ~40 ns
// whatever its size: sixteen row copies per stage capped Q6_K at 87 % of the copy peak and held the 32-column
// formats at 3.0-3.4 TB/s.
struct Geom { int kseg, segb, rs, box_bytes, pitch; };
// words of a 256-column group in memory, and words of a box row in the stage
__host__ __device__ constexpr int box3_words(int dt) {
  return dt == DT_Q4_K || dt == DT_Q4_0 ? 36 : dt == DT_Q5_K || dt == DT_Q5_0 ? 44 : dt == DT_Q5_1 ? 48 : dt == DT_Q4_1 ? 40 : dt == DT_Q8_0 ? 68 : 0;
}
__host__ __device__ constexpr int box3_pitch_words(int dt) { return dt == DT_Q5_1 ? 52 : dt == DT_Q4_1 ? 44 : box3_words(dt); }
__host__ __device__ constexpr int box3_kseg(int dt) { return dt == DT_Q4_K || dt == DT_Q4_0 ? 4096 : 2048; }
static_assert(Fmt<DT_Q4_K>::KSEG == box3_kseg(DT_Q4_K) && Fmt<DT_Q5_K>::KSEG == box3_kseg(DT_Q5_K) && Fmt<DT_Q4_0>::KSEG == box3_kseg(DT_Q4_0) &&
              Fmt<DT_Q5_0>::KSEG == box3_kseg(DT_Q5_0) && Fmt<DT_Q8_0>::KSEG == box3_kseg(DT_Q8_0) && Fmt<DT_Q5_1>::KSEG == box3_kseg(DT_Q5_1) && Fmt<DT_Q4_1>::KSEG == box3_kseg(DT_Q4_1), "stage length");
__host__ __device__ constexpr int box3_bytes(int dt) { return box3_kseg(dt) / 256 * 16 * box3_pitch_words(dt) * 4; }
static_assert(box3_bytes(DT_Q4_K) <= MAX_CHUNK && box3_bytes(DT_Q5_K) <= MAX_CHUNK && box3_bytes(DT_Q4_0) <= MAX_CHUNK &&
              box3_bytes(DT_Q5_0) <= MAX_CHUNK && box3_bytes(DT_Q8_0) <= MAX_CHUNK && box3_bytes(DT_Q5_1) <= MAX_CHUNK && box3_bytes(DT_Q4_1) <= MAX_CHUNK, "ring stage");
__device__ __forceinline__ Geom geom_of(int dtype) {
  if (box3_words(dtype)) return {box3_kseg(dtype), 0, 0, box3_bytes(dtype), 4 * box3_pitch_words(dtype)};
  return {Fmt<DT_Q6_K>::KSEG, Lay<DT_Q6_K, 1>::SEGB, Lay<DT_Q6_K, 1>::RS, 16 * Lay<DT_Q6_K, 1>::SEGB, 0};
}
static_assert(Lay<DT_Q6_K, 1>::RS == Lay<DT_Q6_K, 1>::SEGB, "Q6_K rows lie densely in a stage");

__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
// Bounded wait on a barrier of this CTA; false when it gave up.  Inside a program another warp of the CTA may itself
// be waiting (bounded by the executor's poll limit) for another CTA or another GPU, and that wait can legitimately
// outlast SPIN_LIMIT: with an abort word this wait therefore gives up when the run's abort word is raised (some wait
// of the run ran out) and otherwise only after a hard bound far beyond any poll limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, const unsigned long long* abort_word = nullptr,
                                          unsigned long long epoch = 0) {
  int spins = 0;
  while (!mbar_try_wait(b, parity)) {
    ++spins;
    if (!abort_word) {
      if (spins > SPIN_LIMIT) return false;
    } else if ((spins & 0xffff) == 0) {
      unsigned long long a;
      asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(a) : "l"(abort_word) : "memory");
      if (a == epoch || spins > 256 * SPIN_LIMIT / 4) return false;
    }
  }
  return true;
}
// Q4_K stages lie [block][row][144 bytes]: rows 144 bytes apart are 16 bytes apart modulo
// 128, so the 8-byte fragment reads of four consecutive rows (one half-warp) would overlap in
// the banks.  Fragment row g therefore reads tile row 2 (g & 3) + (g >> 2): the four rows of a
// half-warp are 288 bytes apart (32 modulo 128) and cover all banks once.
__device__ __forceinline__ int q4k_row(int g) { return 2 * (g & 3) + (g >> 2); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory"); }

// What a launch works on: a list of entries in global memory (program) or one entry
// passed by value (single product).
struct Work {
  const ProgEntry* entries;
  const ProgPhase* phases;
  int n_phases;
  const PeerTable* peers;  // row-sharded programs only
  HostOut host;            // single products that deliver their result to the host themselves
  const CUtensorMap* maps; // one per entry (Q4_K, Q6_K; unused for Q8_0)
  int n_entries;           // entries of the program
  uint32_t tag_base;       // tag of phase p in this run = tag_base + p
  int poll_limit;          // bound of the waits on other CTAs' or ranks' data
  const int* sel;          // select programs: entry E reads its weights through maps[E.map_base + sel[E.sel_slot]]
};
// Slots of the counter array beside the per-phase counters ([0, 4095) this rank's CTAs per phase,
// [4096, 8191) arrivals of the peers per phase).
constexpr int TAG_SLOT = 4095;                          // first tag the next run may use (read at creation)
constexpr int ABORT_SLOT = PEER_COUNTER_OFFSET + 4095;  // epoch of a run in which a wait ran out

// Tile range of this CTA inside a phase, and inside one entry of it.
// The grid is two CTAs per SM and CTAs b and b + nb/2 usually share an SM.  Slices are dealt so
// that those two get neighbouring slices: the slices with one tile more than the rest (or one
// less) then spread over the SMs instead of meeting in pairs on a few of them.
__device__ __forceinline__ void phase_range(const ProgPhase& P, int bid, int nb, int* lo, int* hi) {
  const int half = nb >> 1;
  const int slot = (nb & 1) ? bid : (bid < half ? 2 * bid : 2 * (bid - half) + 1);
  *lo = (int)((int64_t)P.n_tiles * slot / nb);
  *hi = (int)((int64_t)P.n_tiles * (slot + 1) / nb);
}
__device__ __forceinline__ bool entry_range(const ProgEntry& E, int lo, int hi, int* t0, int* t1) {
  *t0 = max(lo, E.tile_begin) - E.tile_begin;
  *t1 = min(hi, E.tile_begin + E.n_tiles) - E.tile_begin;
  return *t0 < *t1;
}

// Everything between "the input exists" and "its digit planes are in shared memory": the 1/rms of an
// RMSNorm input (all consumer warps, when need_rms) and this warp's share of the activation split.
// Not inlined: it runs once per entry and span, and its registers (sixteen pairs in flight per lane)
// must not compete with the accumulators of the block routines.
#ifndef LLR_PREP_INLINE
#define LLR_PREP_INLINE __forceinline__
#endif
template <int MT, bool PEERS, bool FLOW>
__device__ LLR_PREP_INLINE bool prepare_activations(const XSrc src, int cols, int tokens, float eps, int span, int nblk256, bool need_rms,
                                                 uint8_t* dig, float* sxf, float* xsi, float* s_part, float* s_inv, WaitCtx wc) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t keep = l2_policy_evict_last();
  if (FLOW && need_rms) row_inv_rms<MT, PEERS>(src, cols, tokens, eps, s_part, s_inv, warp, lane, wc, keep);
  split_activations<MT, PEERS, FLOW>(src, cols, span * Sp<MT>::SPAN, nblk256, tokens, dig, sxf, xsi, s_inv, warp, lane, wc, keep);
  return wc.dead;
}

// What the digit planes in shared memory were made from; kept in shared memory, one record per consumer
// warp (warps pass an entry at different times), because it is looked at once per entry and span and
// would otherwise occupy registers throughout the block routines.
struct SplitKey {
  const void* x;
  const void* x2;
  int cols, span, tokens, op, ph, pad;
};

// DTFIX: the one format of a single-product launch (the other block routines are compiled
// out, which keeps the consumers under the register budget of two CTAs per SM), or -1 for
// programs, which switch per entry.
// FLOW: the program may carry results from entry to entry as tagged pairs and apply RMSNorm / SwiGLU /
// residual adds; compiled out otherwise (the plain split and the per-phase counters need fewer registers
// around the block routines, which run at the register limit of two CTAs per SM).
// SELECT: one-phase programs whose entries choose their matrix at run time (see Work::sel); the table is written by an
// earlier kernel of the stream, so the producer too waits for that kernel before it fetches anything.
template <int MT, bool PROGRAM, int DTFIX, bool PEERS = false, bool HOSTOUT = false, bool FLOW = false, bool SELECT = false>
__device__ __forceinline__ void stream_body(const Work wk, unsigned long long* counters,
                                            unsigned long long epoch, int* err) {
  using L = SLay<MT>;
  constexpr int NT = L::NT;
  constexpr int SPAN = Sp<MT>::SPAN;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem + L::RING;
  uint8_t* dig = smem + L::DIG;
  float* sxf = (float*)(smem + L::SXF);
  float* xsi = (float*)(smem + L::XSI);
  float* red = (float*)(smem + L::RED);
  uint64_t* full = (uint64_t*)(smem + L::BAR);
  uint64_t* empty = full + NST;
  const unsigned long long* abort_word = PROGRAM && counters ? counters + ABORT_SLOT : nullptr;
  uint64_t* rfull = empty + NST;
  uint64_t* rempty = rfull + NRB;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bid = blockIdx.x, nb = gridDim.x;

  // Programmatic dependent launch (single products and one-phase programs are launched that way; elsewhere both
  // instructions do nothing): the next kernel of the stream may be placed now, and this kernel's producer starts
  // streaming weights while the kernel before it still runs; what touches activations or results waits below.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tid == 0) {
    for (int s = 0; s < NST; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CW); }
    for (int s = 0; s < NRB; ++s) { mbar_init(&rfull[s], CW); mbar_init(&rempty[s], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < Sp<MT>::PLANES * Sp<MT>::DS / 16; i += NTHREADS) ((uint4*)dig)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();

  if (warp == CW) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      int c = 0;
      bool ok = true;
      const uint64_t stream_once = l2_policy_evict_first();
      if (SELECT) asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int ph = 0; ph < wk.n_phases; ++ph) {
        const ProgPhase P = wk.phases[ph];
        int lo, hi;
        phase_range(P, bid, nb, &lo, &hi);
        for (int ei = 0; ei < P.n_entries && lo < hi; ++ei) {
          const ProgEntry& E = wk.entries[P.first_entry + ei];
          int t0, t1;
          if (!entry_range(E, lo, hi, &t0, &t1)) continue;
          const int dtype = DTFIX >= 0 ? DTFIX : E.dtype;
          const Geom gm = geom_of(dtype);
          const CUtensorMap* map = SELECT ? wk.maps + E.map_base + wk.sel[E.sel_slot] : wk.maps + (PROGRAM ? P.first_entry + ei : 0);
          const int cols = E.cols;
          const int n_span = (cols + SPAN - 1) / SPAN;
          for (int span = 0; span < n_span; ++span) {
            const int span_cols = min(SPAN, cols - span * SPAN);
            const int nsub = (span_cols + gm.kseg - 1) / gm.kseg;
            for (int tile = t0; tile < t1; ++tile) {
              for (int sub = 0; sub < nsub; ++sub, ++c) {
                const int stage = c % NST;
                if (ok && !mbar_wait(&empty[stage], (uint32_t)(((c / NST) & 1) ^ 1), abort_word, epoch)) { ok = false; report_error(err, 1); }
                uint8_t* dst = ring + stage * MAX_CHUNK;
                const int seg = span * (SPAN / gm.kseg) + sub;
                // rows and groups beyond the matrix are filled with zeros and still counted
                mbar_expect_tx(&full[stage], (uint32_t)gm.box_bytes);
                if (dtype != DT_Q6_K) tma_box_3d(dst, map, 0, tile * 16, seg * (gm.kseg / 256), &full[stage], stream_once);
                else tma_box_2d(dst, map, seg * (Lay<DT_Q6_K, 1>::SEGB / 8), tile * 16, &full[stage], stream_once);
              }
            }
          }
        }
      }
    }
    return;
  }

  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == CW + 1) {
    // -------------------------------------------------------------- reducer
    int j = 0;  // tiles reduced by this CTA
    bool ok = true;
    WaitCtx wc{err, counters ? counters + ABORT_SLOT : nullptr, epoch, wk.poll_limit, false};
    for (int ph = 0; ph < wk.n_phases; ++ph) {
      const ProgPhase P = wk.phases[ph];
      int lo, hi;
      phase_range(P, bid, nb, &lo, &hi);
      for (int ei = 0; ei < P.n_entries && lo < hi; ++ei) {
        const ProgEntry E = wk.entries[P.first_entry + ei];
        int t0, t1;
        if (!entry_range(E, lo, hi, &t0, &t1)) continue;
        const int n_span = (E.cols + SPAN - 1) / SPAN;
        for (int span = 0; span < n_span; ++span) {
          const int n_part = (min(SPAN, E.cols - span * SPAN) + PART_COLS - 1) / PART_COLS;
          float carry[(16 * MT + 31) / 32];
          for (int tile = t0; tile < t1; ++tile)
          for (int part = 0; part < n_part; ++part, ++j) {
            const int rb = j % NRB;
            if (ok && !mbar_wait(&rfull[rb], (uint32_t)((j / NRB) & 1), abort_word, epoch)) { ok = false; if (lane == 0) report_error(err, 1); }
            const float* rp0 = red + rb * CW * 16 * MT;
#pragma unroll
            for (int slot = 0; slot < (16 * MT + 31) / 32; ++slot) {
              const int idx = lane + 32 * slot;
              if (idx >= 16 * MT) break;
              const int r = idx / MT, k = idx % MT, row = tile * 16 + r;
              const bool valid = row < E.rows && k < E.tokens;
              const int64_t at = (int64_t)k * E.y_ld + row;
              float* yp = E.y + at;
              float v = 0.f;
#pragma unroll
              for (int w = 0; w < CW; ++w) v += rp0[w * 16 * MT + idx];
              // y = ((P0 + P1) + P2) + ...: the parts of a span are chained in a register, the spans through y
              if (part != 0) v += carry[slot];
              else if (span != 0 && valid) v += *yp;
              if (part != n_part - 1) { carry[slot] = v; continue; }
              if (valid) {
                if (span != n_span - 1) { *yp = v; continue; }
                if (FLOW && E.resid) {  // residual add: result + residual, as the walk adds them (decode.rs:2938, :3050)
                  if (E.resid_phase >= 0) {
                    const uint2* rp = (const uint2*)E.resid + at;
                    unsigned long long a = ld_pair<PEERS>(rp);
                    if ((uint32_t)(a >> 32) != wk.tag_base + (uint32_t)E.resid_phase && !wc.dead) {
                      poll_pair<PEERS>(rp, wk.tag_base + (uint32_t)E.resid_phase, wc);
                      a = ld_pair<PEERS>(rp);
                    }
                    v = __fadd_rn(v, __uint_as_float((uint32_t)a));
                  } else {
                    v = __fadd_rn(v, ((const float*)E.resid)[at]);
                  }
                }
                *yp = v;
                if (HOSTOUT) *(float*)((char*)yp + wk.host.y_delta) = v;
                if (FLOW && E.yt) st_pair<false>((uint2*)E.yt + at, v, wk.tag_base + (uint32_t)ph);
                if (PEERS) {
                  const int np = wk.peers->n_peers;
                  for (int p = 0; p < np; ++p) {
                    *(float*)((char*)yp + wk.peers->y_delta[p]) = v;
                    if (FLOW && E.yt) st_pair<true>((char*)((uint2*)E.yt + at) + wk.peers->y_delta[p], v, wk.tag_base + (uint32_t)ph);
                  }
                }
              }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&rempty[rb]);
          }
        }
      }
      if (PROGRAM && (P.wait_prev & 2)) {
        // this CTA's share of the phase is written and a later phase waits for the counter: publish it
        if (PEERS) {
          // One signal per rank and phase crosses NVLink, not one per CTA (hundreds of remote atomics
          // on one word serialise at tens of nanoseconds each): CTAs count locally, and the CTA
          // that completes the local count tells every peer.
          // Ordering: the lanes' peer stores -> __syncwarp -> lane 0's gpu-scope release on the
          // local counter -> (last CTA) acquire of everybody's releases -> system-scope release
          // to the peers.  Releases are cumulative, so one system-scope fence per rank and phase
          // (inside the last CTA's red.release.sys) covers every CTA's peer stores.
          __syncwarp();
          if (lane == 0) {
            unsigned long long old;
            asm volatile("atom.acq_rel.gpu.global.add.u64 %0, [%1], %2;" : "=l"(old) : "l"(counters + ph), "l"(1ull) : "memory");
            if (old + 1 == epoch * (unsigned long long)nb) {  // the release of the add below is cumulative
              const int np = wk.peers->n_peers;
              for (int p = 0; p < np; ++p)
                asm volatile("red.release.sys.global.add.u64 [%0], %1;"
                             ::"l"(wk.peers->counters[p] + PEER_COUNTER_OFFSET + ph), "l"(1ull) : "memory");
            }
          }
        } else {
          __syncwarp();
          if (lane == 0)  // release: the y values written above are visible before the count
            asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(counters + ph), "l"(1ull) : "memory");
        }
      }
    }
    if (HOSTOUT) {
      // this CTA's stores to host memory are performed; the CTA that counts last tells the host
      __threadfence_system();
      __syncwarp();
      if (lane == 0) {
        unsigned int old;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(wk.host.count) : "memory");
        if (old + 1 == (unsigned int)nb) {
          *wk.host.count = 0;  // the next launch counts from zero; its reducers run after this grid has completed
          __threadfence_system();
          *(volatile int*)wk.host.done = wk.host.ticket;
        }
      }
    }
    return;
  }

  // ---------------------------------------------------------------- consumers
  const int g = lane >> 2, t = lane & 3;
  int c = 0, j = 0;
  bool ok = true;
  __shared__ SplitKey s_key[CW];
  if (lane == 0) s_key[warp] = SplitKey{nullptr, nullptr, -1, -1, -1, -1, -1, 0};
  __syncwarp();
  bool dead = false;  // a wait of this warp ran out, or another CTA said so: later waits return at once
  // Programs: the entries of a phase are fetched into shared memory before the dependency
  // wait, so that after the wait the consumers do not pay a global-memory round trip for them.
  constexpr int ENT_CACHE = 4, ENT_WORDS = sizeof(ProgEntry) / 8;
  __shared__ __align__(16) unsigned long long s_ent[2][ENT_CACHE][ENT_WORDS];
  __shared__ float s_part[CW * 8], s_inv[8];
  __shared__ __align__(16) ProgPhase s_phase[2];
  // Programs: phase descriptors and the first entries of a phase reach shared memory one phase ahead
  // (asynchronous copies issued by warp 0 while the previous phase is being computed), so that a new
  // phase starts without a round trip to global memory for its own description.
  auto prefetch_phase = [&](int q, int first_entry) {  // warp 0: phase q, whose entries start at first_entry
    if (lane == 0) cp_async16(&s_phase[q & 1], wk.phases + q);
    const int chunk = lane;  // 32 chunks of 16 bytes = ENT_CACHE entries of 128 bytes
    if (first_entry + chunk / 8 < wk.n_entries)
      cp_async16((char*)&s_ent[q & 1][0][0] + 16 * chunk, (const char*)(wk.entries + first_entry) + 16 * chunk);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  static_assert(ENT_CACHE * sizeof(ProgEntry) == 32 * 16, "one 16-byte chunk per lane");
  if (PROGRAM && warp == 0) prefetch_phase(0, 0);
  for (int ph = 0; ph < wk.n_phases; ++ph) {
    if (PROGRAM) {
      if (warp == 0) asm volatile("cp.async.wait_group 0;" ::: "memory");
      consumer_sync();  // publish the descriptor and the cached entries of this phase
    }
    const ProgPhase P = PROGRAM ? s_phase[ph & 1] : wk.phases[ph];
    // everybody is in phase ph now: the buffers of phase ph - 1 are free for phase ph + 1
    if (PROGRAM && warp == 0 && ph + 1 < wk.n_phases) prefetch_phase(ph + 1, P.first_entry + P.n_entries);
    int lo, hi;
    phase_range(P, bid, nb, &lo, &hi);
    const int n_cached = PROGRAM ? min(P.n_entries, ENT_CACHE) : 0;
    // Counter dependencies (strict phases with an input that is not a result of the program) are
    // awaited as late as possible: everything that does not need the activations (entry, geometry)
    // is done first, so that the loads of the split are the first thing after the wait.  A CTA
    // without tiles in the phase does not wait at all: the counters it waits for in its next
    // phase imply this one.  Tagged inputs need none of this: their loads are the wait.
    // A sharded program with counters also holds back the first phase of a run until every rank
    // has finished the previous run (its peers' stores into this rank's buffers belong to that run).
    bool waited = !(PROGRAM && (((P.wait_prev & 1) && ph > 0) || (PEERS && ph == 0 && (P.wait_prev & 4))));
    for (int ei = 0; ei < P.n_entries && lo < hi; ++ei) {
      const ProgEntry& Eref = ei < n_cached ? *(const ProgEntry*)&s_ent[ph & 1][ei][0] : wk.entries[P.first_entry + ei];
      const ProgEntry E = Eref;  // a copy: fields stay in registers across the waits below (those clobber memory)
      int t0, t1;
      if (!entry_range(E, lo, hi, &t0, &t1)) continue;
      const Geom gm = geom_of(DTFIX >= 0 ? DTFIX : E.dtype);
      const int n_span = (E.cols + SPAN - 1) / SPAN;
      const void* xkey = FLOW && E.xt ? E.xt : (const void*)E.x;
      for (int span = 0; span < n_span; ++span) {
        const int span_cols = min(SPAN, E.cols - span * SPAN), nblk256 = span_cols >> 8;
        // (a buffer may be rewritten by a later phase: digit planes are never carried across phases)
        const SplitKey have = s_key[warp];
        if (!waited || have.x != xkey || have.cols != E.cols || have.span != span || have.tokens != E.tokens ||
            (PROGRAM && have.ph != ph) || (FLOW && (have.op != E.x_op || have.x2 != E.x2))) {
          if (!waited) {
            if (tid == 0 && !dead) {
              const unsigned long long runs = ph > 0 ? epoch : epoch - 1;
              const unsigned long long want = runs * (unsigned long long)nb;
              const int dep = ph > 0 ? ph - 1 : wk.n_phases - 1;
              const unsigned long long* cp = counters + dep;
              // sharded: also one arrival per peer and run on this rank's copy of the peers' counter
              const unsigned long long want_peers = PEERS ? runs * (unsigned long long)wk.peers->n_peers : 0ull;
              const unsigned long long* pp = counters + PEER_COUNTER_OFFSET + dep;
              int polls = 0;
              for (;;) {
                unsigned long long v, u = want_peers;
                asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(cp) : "memory");
                if (PEERS) asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(u) : "l"(pp) : "memory");
                if (v >= want && (!PEERS || u >= want_peers)) break;
                if ((polls & 15) == 15 && ld_pair<false>(counters + ABORT_SLOT) == epoch) break;
                if (++polls > wk.poll_limit) {
                  *(volatile unsigned long long*)(counters + ABORT_SLOT) = epoch;
                  report_error(err, 2);
                  break;
                }
                __nanosleep(polls < 8 ? 64 : 256);  // hundreds of CTAs poll one word: keep the L2 bank free for the adds
              }
            }
            consumer_sync();
            waited = true;
          }
          // the planes a warp overwrites are the ones it alone reads (see split_activations)
          __syncwarp();
          // the 1/rms of the row belongs to the whole row: computed when its first span is split
          const bool need_rms = FLOW && E.x_op == XOP_RMSNORM && span == 0;
          XSrc src{E.x, nullptr, nullptr, 0u, 0u, XOP_NONE, 0};
          if (FLOW) {
            src.xt = (const uint2*)E.xt;
            src.x2 = E.x2;
            src.tag = wk.tag_base + (uint32_t)E.x_phase;
            src.tag2 = wk.tag_base + (uint32_t)E.x2_phase;
            src.op = E.x_op;
            src.x2_tagged = E.x2_phase >= 0;
          }
          dead = prepare_activations<MT, PEERS, FLOW>(src, E.cols, E.tokens, FLOW ? E.eps : 0.f, span, nblk256, need_rms, dig, sxf, xsi,
                                                s_part, s_inv, WaitCtx{err, PROGRAM ? counters + ABORT_SLOT : nullptr, epoch, wk.poll_limit, dead});
          if (lane == 0) s_key[warp] = SplitKey{xkey, FLOW ? E.x2 : nullptr, E.cols, span, E.tokens, FLOW ? E.x_op : 0, ph, 0};
          __syncwarp();
        }
        const int nsub = (span_cols + gm.kseg - 1) / gm.kseg;
        // Partial sums go to the reducer every PART_COLS columns, whatever the span: a row's result is then formed
        // the same way for one activation row (whose span is twice as long) as inside a batch.
        const int part_mask = PART_COLS / gm.kseg - 1;  // stages per part minus one: 0 or 1
        for (int tile = t0; tile < t1; ++tile) {
          AccT<MT> acc;
          auto clear = [&] {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int i = 0; i < 4; ++i) acc.y[nt][i] = 0.f;
#pragma unroll
            for (int k = 0; k < MT; ++k) acc.mn[0][k] = acc.mn[1][k] = 0.f;
          };
          clear();
          for (int sub = 0; sub < nsub; ++sub, ++c) {
            const int stage = c % NST;
            if (ok && !mbar_wait(&full[stage], (uint32_t)((c / NST) & 1), abort_word, epoch)) { ok = false; if (lane == 0) report_error(err, 1); }
            const uint8_t* chunk = ring + stage * MAX_CHUNK;
            const uint8_t* rowA = chunk + g * gm.rs;
            const uint8_t* rowB = chunk + (g + 8) * gm.rs;
            const int seg_cols = min(gm.kseg, span_cols - sub * gm.kseg);
            const int dtype = DTFIX >= 0 ? DTFIX : E.dtype;
            if (dtype == DT_Q4_K) {
              // stage layout [block][row][144]; fragment row g is tile row q4k_row(g), see there
              for (int b = warp; b < (seg_cols >> 8); b += CW)
                block_q4k<MT>(chunk + (b * 16 + q4k_row(g)) * 144, chunk + (b * 16 + q4k_row(g) + 8) * 144, sub * (gm.kseg / 256) + b, dig, sxf, xsi, g, t, acc);
            } else if (DTFIX == DT_Q5_K) {  // single products only, like the nibble formats below
              for (int b = warp; b < (seg_cols >> 8); b += CW)
                block_q4k<MT, true>(chunk + (b * 16 + q4k_row(g)) * 176, chunk + (b * 16 + q4k_row(g) + 8) * 176, sub * (gm.kseg / 256) + b, dig, sxf, xsi, g, t, acc);
            } else if (dtype == DT_Q6_K) {
              for (int b = warp; b < (seg_cols >> 8); b += CW)
                block_q6k<MT>(rowA, rowB, b, sub * (gm.kseg / 256) + b, dig, xsi, g, t, acc);
            } else if (DTFIX == DT_Q4_0) {  // the nibble formats run as single products only (never inside programs)
              for (int b8 = warp; b8 < (seg_cols >> 8); b8 += CW) {
                float xw[NT];
                group_scales<MT>(xsi, sub * (gm.kseg / 256) + b8, t, (t & 1) ? 4096.f : 0.0625f, xw);
                const uint8_t* grpA = chunk + (b8 * 16 + q4k_row(g)) * gm.pitch;  // stage layout [group][row][pitch]
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  block_q40<MT>(grpA, grpA + 8 * gm.pitch, i, sub * (gm.kseg / 32) + b8 * 8 + i, dig, xw, g, t, acc);
              }
            } else if (DTFIX == DT_Q5_0) {
              for (int b8 = warp; b8 < (seg_cols >> 8); b8 += CW) {
                float xw[NT];
                group_scales<MT>(xsi, sub * (gm.kseg / 256) + b8, t, (t & 1) ? 8192.f : 0.125f, xw);
                const uint8_t* grpA = chunk + (b8 * 16 + q4k_row(g)) * gm.pitch;  // stage layout [group][row][pitch]
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  block_q50<MT>(grpA, grpA + 8 * gm.pitch, i, sub * (gm.kseg / 32) + b8 * 8 + i, dig, sxf, xw, g, t, acc);
              }
            } else if (DTFIX == DT_Q5_1) {
              for (int b8 = warp; b8 < (seg_cols >> 8); b8 += CW) {
                float xw[NT];
                group_scales<MT>(xsi, sub * (gm.kseg / 256) + b8, t, (t & 1) ? 65536.f : 1.f, xw);
                const uint8_t* grpA = chunk + (b8 * 16 + q4k_row(g)) * gm.pitch;  // stage layout [group][row][pitch]
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  block_q51<MT>(grpA, grpA + 8 * gm.pitch, i, sub * (gm.kseg / 32) + b8 * 8 + i, dig, sxf, xw, g, t, acc);
              }
            } else if (DTFIX == DT_Q4_1) {
              for (int b8 = warp; b8 < (seg_cols >> 8); b8 += CW) {
                float xw[NT];
                group_scales<MT>(xsi, sub * (gm.kseg / 256) + b8, t, (t & 1) ? 65536.f : 1.f, xw);
                const uint8_t* grpA = chunk + (b8 * 16 + q4k_row(g)) * gm.pitch;  // stage layout [group][row][pitch]
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  block_q41<MT>(grpA, grpA + 8 * gm.pitch, i, sub * (gm.kseg / 32) + b8 * 8 + i, dig, sxf, xw, g, t, acc);
              }
            } else {
              for (int b8 = warp; b8 < (seg_cols >> 8); b8 += CW) {
                float xw[NT];
                group_scales<MT>(xsi, sub * (gm.kseg / 256) + b8, t, (t & 1) ? 65536.f : 1.f, xw);
                const uint8_t* grpA = chunk + (b8 * 16 + q4k_row(g)) * gm.pitch;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  block_q80<MT>(grpA, grpA + 8 * gm.pitch, i, sub * (gm.kseg / 32) + b8 * 8 + i, dig, xw, g, t, acc);
              }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);  // this warp no longer reads the stage
            if ((sub & part_mask) != part_mask && sub != nsub - 1) continue;
          // ---- hand this warp's partial sums of the part to the reducer ----
          const int rb = j % NRB;
          if (ok && !mbar_wait(&rempty[rb], (uint32_t)(((j / NRB) & 1) ^ 1), abort_word, epoch)) { ok = false; if (lane == 0) report_error(err, 1); }
          float* myred = red + (rb * CW + warp) * 16 * MT;
          if ((DTFIX >= 0 ? DTFIX : E.dtype) == DT_Q4_K || DTFIX == DT_Q5_1 || DTFIX == DT_Q4_1 || DTFIX == DT_Q5_K) {
#pragma unroll
            for (int k = 0; k < MT; ++k)
#pragma unroll
              for (int r = 0; r < 2; ++r) {
                float v = acc.mn[r][k];
                v += __shfl_xor_sync(~0u, v, 1);
                v += __shfl_xor_sync(~0u, v, 2);
                acc.mn[r][k] = v;
              }
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            float vA = acc.y[nt][0] + acc.y[nt][1], vB = acc.y[nt][2] + acc.y[nt][3];
            vA += __shfl_xor_sync(~0u, vA, 1);
            vB += __shfl_xor_sync(~0u, vB, 1);
            const int tok = 2 * nt + (t >> 1);
            if ((t & 1) == 0 && tok < MT) {
              float mA = 0.f, mB = 0.f;
#pragma unroll
              for (int k = 0; k < MT; ++k)
                if (k == tok) { mA = acc.mn[0][k]; mB = acc.mn[1][k]; }
              const int gr = box3_words(DTFIX >= 0 ? DTFIX : E.dtype) ? q4k_row(g) : g;  // box stages hold the rows in that order
              myred[gr * MT + tok] = vA - mA;
              myred[(gr + 8) * MT + tok] = vB - mB;
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&rfull[rb]);
          ++j;
          clear();
          }
        }
      }
    }
  }
}

// two CTAs per SM need <= 102 registers per thread; with more than two activation rows the
// digit planes leave room for one CTA only
template <int MT, int DT>
__global__ void __launch_bounds__(NTHREADS, (MT <= 2 ? 2 : 1))
gemv_stream_kernel(const __grid_constant__ ProgEntry one, const __grid_constant__ CUtensorMap map, int* __restrict__ err) {
  __shared__ ProgPhase phase;
  if (threadIdx.x == 0) phase = ProgPhase{0, 1, one.n_tiles, 0};
  __syncthreads();
  Work wk{&one, &phase, 1, nullptr, HostOut{}, &map, 1, 0u, 0};
  stream_body<MT, false, DT>(wk, nullptr, 0ull, err);
}

template <int MT, int DT>
__global__ void __launch_bounds__(NTHREADS, (MT <= 2 ? 2 : 1))
gemv_stream_hostout_kernel(const __grid_constant__ ProgEntry one, const __grid_constant__ CUtensorMap map,
                           const __grid_constant__ HostOut ho, int* __restrict__ err) {
  __shared__ ProgPhase phase;
  if (threadIdx.x == 0) phase = ProgPhase{0, 1, one.n_tiles, 0};
  __syncthreads();
  Work wk{&one, &phase, 1, nullptr, ho, &map, 1, 0u, 0};
  stream_body<MT, false, DT, false, true>(wk, nullptr, 0ull, err);
}

// One product with one activation row whose matrix is chosen on the device: maps[*sel] of an array of tensor maps
// of equally shaped matrices (the experts of a routed layer; the kernels address weights through the map alone).
// *sel is written by an earlier kernel of the stream, so nothing is fetched before that kernel has finished.
template <int DT>
__global__ void __launch_bounds__(NTHREADS, 2)
gemv_stream_select_kernel(const __grid_constant__ ProgEntry one, const CUtensorMap* __restrict__ maps, const int* __restrict__ sel,
                          int* __restrict__ err) {
  __shared__ ProgPhase phase;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) phase = ProgPhase{0, 1, one.n_tiles, 0};
  __syncthreads();
  Work wk{&one, &phase, 1, nullptr, HostOut{}, maps + *sel, 1, 0u, 0};
  stream_body<1, false, DT>(wk, nullptr, 0ull, err);
}

// What changes from run to run of a program.
struct RunArgs {
  unsigned long long epoch;     // runs of this program so far, this one included (what the counters count in)
  unsigned long long tag_next;  // first tag after this run's
  uint32_t tag_base;
  int poll_limit;
  int n_entries;
};

// (FLOW kernels keep sixteen tagged pairs per lane in flight and carry the element-wise operations: they do not
// fit the 96 registers of two CTAs per SM without spilling into the block routines, so they run one CTA per SM.)
template <int MT, bool FLOW>
__global__ void __launch_bounds__(NTHREADS, (MT <= 2 && !FLOW ? 2 : 1))
gemv_program_kernel(const ProgEntry* __restrict__ entries, const ProgPhase* __restrict__ phases, int n_phases,
                    const CUtensorMap* __restrict__ maps, unsigned long long* __restrict__ counters,
                    const RunArgs run, int* __restrict__ err) {
  Work wk{entries, phases, n_phases, nullptr, HostOut{}, maps, run.n_entries, run.tag_base, run.poll_limit};
  if (blockIdx.x == 0 && threadIdx.x == 0) counters[TAG_SLOT] = run.tag_next;
  stream_body<MT, true, -1, false, false, FLOW>(wk, counters, run.epoch, err);
}

template <int MT, bool FLOW>
__global__ void __launch_bounds__(NTHREADS, (MT <= 2 && !FLOW ? 2 : 1))
gemv_sharded_program_kernel(const ProgEntry* __restrict__ entries, const ProgPhase* __restrict__ phases, int n_phases,
                            const CUtensorMap* __restrict__ maps, unsigned long long* __restrict__ counters,
                            const RunArgs run, const PeerTable* __restrict__ peers, int* __restrict__ err) {
  Work wk{entries, phases, n_phases, peers, HostOut{}, maps, run.n_entries, run.tag_base, run.poll_limit};
  if (blockIdx.x == 0 && threadIdx.x == 0) counters[TAG_SLOT] = run.tag_next;
  stream_body<MT, true, -1, true, false, FLOW>(wk, counters, run.epoch, err);
}

// One phase of one-token products that each pick one of several equally shaped matrices through a device table.
__global__ void __launch_bounds__(NTHREADS, 2)
gemv_select_program_kernel(const ProgEntry* __restrict__ entries, const ProgPhase* __restrict__ phases,
                           const CUtensorMap* __restrict__ maps, const int* __restrict__ sel,
                           unsigned long long* __restrict__ counters, const RunArgs run, int* __restrict__ err) {
  Work wk{entries, phases, 1, nullptr, HostOut{}, maps, run.n_entries, run.tag_base, run.poll_limit, sel};
  if (blockIdx.x == 0 && threadIdx.x == 0) counters[TAG_SLOT] = run.tag_next;
  stream_body<1, true, -1, false, false, false, true>(wk, counters, run.epoch, err);
}

// Tensor map of one matrix for the stage loads (see Geom).
bool encode_weight_map(const uint8_t* w, int dtype, int64_t rows, int64_t cols, int64_t row_bytes, CUtensorMap* map) {
  memset(map, 0, sizeof(*map));
  if (!box3_words(dtype) && dtype != DT_Q6_K) return true;
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return false;
  const cuuint32_t estr[3] = {1, 1, 1};
  if (box3_words(dtype)) {
    // a box row wider than the group (Q4_1, Q5_1) ends outside the tensor's inner extent: filled with zeros, not read
    const cuuint32_t words = (cuuint32_t)box3_words(dtype);
    const cuuint64_t dims[3] = {words, (cuuint64_t)rows, (cuuint64_t)(cols / 256)};
    const cuuint64_t strides[2] = {(cuuint64_t)row_bytes, 4 * words};
    const cuuint32_t box[3] = {(cuuint32_t)box3_pitch_words(dtype), 16, (cuuint32_t)(box3_kseg(dtype) / 256)};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, (void*)w, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 8), (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(Lay<DT_Q6_K, 1>::SEGB / 8), 16};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, (void*)w, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <class K>
cudaError_t occupancy(K kern, int smem, int* blocks_per_sm) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  int n = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, NTHREADS, smem);
  if (e != cudaSuccess) return e;
  *blocks_per_sm = n > 0 ? n : 1;
  return cudaSuccess;
}

template <int MT, int DT>
cudaError_t launch_single(const MatView& m, const float* x, float* y, int tokens, cudaStream_t stream,
                          int sm_count, int* err, const HostOut* ho) {
  constexpr int smem = SLay<MT>::TOTAL;
  static PerDevice cache, cache_ho;  // per instantiation
  std::atomic<int>& slot = (ho ? cache_ho : cache).here();
  int bps = slot.load(std::memory_order_relaxed);
  if (bps == 0) {
    cudaError_t e = ho ? occupancy(gemv_stream_hostout_kernel<MT, DT>, smem, &bps) : occupancy(gemv_stream_kernel<MT, DT>, smem, &bps);
    if (e != cudaSuccess) return e;
    slot.store(bps, std::memory_order_relaxed);
  }
  ProgEntry E{m.w, x, y, m.row_bytes, (int)m.rows, (int)m.cols, m.dtype, tokens, 0, (int)((m.rows + 15) / 16), m.rows};
  CUtensorMap map;
  if (!encode_weight_map(m.w, m.dtype, m.rows, m.cols, m.row_bytes, &map)) return cudaErrorNotSupported;
  int grid = sm_count * bps;
  if (grid > E.n_tiles) grid = E.n_tiles;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (ho) return cudaLaunchKernelEx(&cfg, gemv_stream_hostout_kernel<MT, DT>, E, map, *ho, err);
  return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<MT, DT>, E, map, err);
}

}  // namespace

bool gemv_mma_supported(const MatView& m) {
  if (m.dtype != DT_Q4_K && m.dtype != DT_Q6_K && m.dtype != DT_Q8_0 && m.dtype != DT_Q4_0 && m.dtype != DT_Q5_0 && m.dtype != DT_Q5_1 &&
      m.dtype != DT_Q4_1 && m.dtype != DT_Q5_K)
    return false;
  if (m.rows <= 0 || m.cols <= 0 || m.rows > (1 << 30) || m.cols > (1 << 30)) return false;
  if (((uintptr_t)m.w & 15) != 0 || m.row_bytes % 16 != 0) return false;
  if (m.cols % 256 != 0) return false;
  // every column piece of a row must start and end on a 16-byte boundary
  if (m.dtype == DT_Q6_K && m.cols % 2048 != 0) return false;
  return true;
}

static cudaError_t launch_passes(const MatView& m, const float* x, float* y, int64_t tokens, cudaStream_t stream,
                                 int sm_count, int* err, uint64_t* launches, const HostOut* ho) {
  for (int64_t t0 = 0; t0 < tokens; t0 += 8) {
    const int nt = (int)(tokens - t0 < 8 ? tokens - t0 : 8);
    const float* xp = x + t0 * m.cols;
    float* yp = y + t0 * m.rows;
    cudaError_t e;
#define LLR_LAUNCH_DT(D)                                                                      \
    (nt == 1 ? launch_single<1, D>(m, xp, yp, nt, stream, sm_count, err, ho)                  \
     : nt == 2 ? launch_single<2, D>(m, xp, yp, nt, stream, sm_count, err, ho)                \
     : nt <= 4 ? launch_single<4, D>(m, xp, yp, nt, stream, sm_count, err, ho)                \
               : launch_single<8, D>(m, xp, yp, nt, stream, sm_count, err, ho))
    if (m.dtype == DT_Q4_K) e = LLR_LAUNCH_DT(DT_Q4_K);
    else if (m.dtype == DT_Q6_K) e = LLR_LAUNCH_DT(DT_Q6_K);
    else if (m.dtype == DT_Q4_0) e = LLR_LAUNCH_DT(DT_Q4_0);
    else if (m.dtype == DT_Q5_0) e = LLR_LAUNCH_DT(DT_Q5_0);
    else if (m.dtype == DT_Q5_1) e = LLR_LAUNCH_DT(DT_Q5_1);
    else if (m.dtype == DT_Q4_1) e = LLR_LAUNCH_DT(DT_Q4_1);
    else if (m.dtype == DT_Q5_K) e = LLR_LAUNCH_DT(DT_Q5_K);
    else e = LLR_LAUNCH_DT(DT_Q8_0);
#undef LLR_LAUNCH_DT
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
  }
  return cudaSuccess;
}

cudaError_t launch_gemv_mma(const MatView& m, const float* x, float* y, int64_t tokens,
                            cudaStream_t stream, int sm_count, int* err, uint64_t* launches) {
  return launch_passes(m, x, y, tokens, stream, sm_count, err, launches, nullptr);
}

cudaError_t gemv_mma_encode_map(const MatView& m, void* map_out) {
  static_assert(sizeof(CUtensorMap) == GEMV_MAP_BYTES, "tensor map size");
  if (!gemv_mma_supported(m)) return cudaErrorInvalidValue;
  return encode_weight_map(m.w, m.dtype, m.rows, m.cols, m.row_bytes, (CUtensorMap*)map_out) ? cudaSuccess : cudaErrorNotSupported;
}

template <int DT>
static cudaError_t launch_select(const MatView& shape, const void* maps_dev, const int* sel_dev, const float* x, float* y,
                                 cudaStream_t stream, int sm_count, int* err) {
  constexpr int smem = SLay<1>::TOTAL;
  static PerDevice cache;
  std::atomic<int>& slot = cache.here();
  int bps = slot.load(std::memory_order_relaxed);
  if (bps == 0) {
    cudaError_t e = occupancy(gemv_stream_select_kernel<DT>, smem, &bps);
    if (e != cudaSuccess) return e;
    slot.store(bps, std::memory_order_relaxed);
  }
  ProgEntry E{nullptr, x, y, shape.row_bytes, (int)shape.rows, (int)shape.cols, shape.dtype, 1, 0, (int)((shape.rows + 15) / 16), shape.rows};
  int grid = sm_count * bps;
  if (grid > E.n_tiles) grid = E.n_tiles;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemv_stream_select_kernel<DT>, E, (const CUtensorMap*)maps_dev, sel_dev, err);
}

cudaError_t launch_gemv_mma_select(const MatView& shape, const void* maps_dev, const int* sel_dev, const float* x, float* y,
                                   cudaStream_t stream, int sm_count, int* err, uint64_t* launches) {
  if (!gemv_mma_supported(shape)) return cudaErrorInvalidValue;
  cudaError_t e;
  switch (shape.dtype) {
    case DT_Q4_K: e = launch_select<DT_Q4_K>(shape, maps_dev, sel_dev, x, y, stream, sm_count, err); break;
    case DT_Q5_K: e = launch_select<DT_Q5_K>(shape, maps_dev, sel_dev, x, y, stream, sm_count, err); break;
    case DT_Q6_K: e = launch_select<DT_Q6_K>(shape, maps_dev, sel_dev, x, y, stream, sm_count, err); break;
    case DT_Q8_0: e = launch_select<DT_Q8_0>(shape, maps_dev, sel_dev, x, y, stream, sm_count, err); break;
    case DT_Q4_0: e = launch_select<DT_Q4_0>(shape, maps_dev, sel_dev, x, y, stream, sm_count, err); break;
    case DT_Q4_1: e = launch_select<DT_Q4_1>(shape, maps_dev, sel_dev, x, y, stream, sm_count, err); break;
    case DT_Q5_0: e = launch_select<DT_Q5_0>(shape, maps_dev, sel_dev, x, y, stream, sm_count, err); break;
    default: e = launch_select<DT_Q5_1>(shape, maps_dev, sel_dev, x, y, stream, sm_count, err); break;
  }
  if (e == cudaSuccess && launches) ++*launches;
  return e;
}

bool gemv_mma_hostout_ok(const MatView& m, int64_t tokens) { return tokens >= 1 && tokens <= 8 && gemv_mma_supported(m); }

cudaError_t launch_gemv_mma_hostout(const MatView& m, const float* x, float* y, int64_t tokens, const HostOut& ho,
                                    cudaStream_t stream, int sm_count, int* err, uint64_t* launches) {
  if (!gemv_mma_hostout_ok(m, tokens)) return cudaErrorInvalidValue;
  return launch_passes(m, x, y, tokens, stream, sm_count, err, launches, &ho);  // one pass
}

// ------------------------------------------------------------------ programs
struct Program {
  ProgEntry* d_entries = nullptr;
  ProgPhase* d_phases = nullptr;
  CUtensorMap* d_maps = nullptr;  // one per entry
  unsigned long long* d_counters = nullptr;  // COUNTER_WORDS words: phase counters, epoch and abort slots
  void* d_tagged = nullptr;       // tagged copies of the results later entries read (single GPU; sharded: in the arena)
  int n_phases = 0, n_entries = 0, max_tokens = 1, grid = 0, counter_phases = 0;
  bool flow = false;  // some entry reads tagged pairs, applies an operation or adds a residual
  unsigned long long epoch = 0;
  unsigned long long tag_next = 1;  // tags are never reused, whatever programs ran on the same buffers before; 0 marks fresh memory
  PeerTable* d_peers = nullptr;   // sharded programs: the peer table, and the counters are not ours
  bool own_counters = true;
  const CUtensorMap* sel_maps = nullptr;  // select programs (program_set_select): the caller's maps and table, both on the device
  const int* sel = nullptr;
};

bool prog_entry_supported(const MatView& m) {
  return (m.dtype == DT_Q4_K || m.dtype == DT_Q6_K || m.dtype == DT_Q8_0) && gemv_mma_supported(m);
}

template <int MT, bool FLOW>
static cudaError_t prog_prepare(int sm_count, int* grid, bool sharded) {
  int bps = 0;
  cudaError_t e = sharded ? occupancy(gemv_sharded_program_kernel<MT, FLOW>, SLay<MT>::TOTAL, &bps)
                          : occupancy(gemv_program_kernel<MT, FLOW>, SLay<MT>::TOTAL, &bps);
  if (e != cudaSuccess) return e;
  if (FLOW) bps = 1;  // see the kernels' launch bounds
  *grid = sm_count * bps;
  return cudaSuccess;
}

template <int MT, bool FLOW>
static cudaError_t prog_launch(Program* p, cudaStream_t stream, int* err, int poll_limit) {
  auto kern = gemv_program_kernel<MT, FLOW>;
  ++p->epoch;
  const ProgEntry* de = p->d_entries;
  const ProgPhase* dp = p->d_phases;
  int np = p->n_phases;
  const CUtensorMap* dm = p->d_maps;
  unsigned long long* dc = p->d_counters;
  // tags of a run: tag_base + phase (32 bits of a counter that only grows; a tag would have to survive
  // 2^32 / phases runs in a buffer that every run rewrites to be mistaken for a new one)
  if ((uint32_t)p->tag_next > 0xffffffffu - (uint32_t)p->n_phases) p->tag_next += 2ull * (unsigned long long)p->n_phases;  // skip the wrap through 0
  RunArgs run{p->epoch, p->tag_next + (unsigned long long)p->n_phases, (uint32_t)p->tag_next, poll_limit, p->n_entries};
  p->tag_next = run.tag_next;
  cudaError_t e;
  // cooperative: every CTA must be resident, the waits between phases are grid-wide dependencies
  if (p->d_peers) {
    const PeerTable* pt = p->d_peers;
    void* args[] = {(void*)&de, (void*)&dp, (void*)&np, (void*)&dm, (void*)&dc, (void*)&run, (void*)&pt, (void*)&err};
    e = cudaLaunchCooperativeKernel((const void*)gemv_sharded_program_kernel<MT, FLOW>, dim3((unsigned)p->grid),
                                    dim3(NTHREADS), args, SLay<MT>::TOTAL, stream);
  } else if (np == 1 && p->counter_phases == 0) {
    // one phase: no CTA waits for another, so the launch need not be cooperative and can overlap its predecessor
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p->grid);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = SLay<MT>::TOTAL;
    cfg.stream = stream;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (MT == 1 && !FLOW && p->sel) e = cudaLaunchKernelEx(&cfg, gemv_select_program_kernel, de, dp, p->sel_maps, p->sel, dc, run, err);
    else e = cudaLaunchKernelEx(&cfg, kern, de, dp, np, dm, dc, run, err);
  } else {
    void* args[] = {(void*)&de, (void*)&dp, (void*)&np, (void*)&dm, (void*)&dc, (void*)&run, (void*)&err};
    e = cudaLaunchCooperativeKernel((const void*)kern, dim3((unsigned)p->grid), dim3(NTHREADS), args,
                                    SLay<MT>::TOTAL, stream);
  }
  if (e != cudaSuccess) {  // nothing ran: counters, tags and the peers stay where they were
    --p->epoch;
    p->tag_next -= (unsigned long long)p->n_phases;
  }
  return e;
}

namespace {
// A result of the program as later entries can address it: the full-width vector (all ranks' rows).
struct Produced {
  const char* base;   // address of row 0, activation row 0
  int64_t ld;         // floats per activation row
  int tokens, phase;
  size_t tagged_off;  // single GPU: byte offset of its tagged copy in Program::d_tagged (SIZE_MAX: none yet)
  bool addressable;   // sharded: ld == world * rows, so the slice's place in the full vector is known
  bool consumed;      // a later entry reads it
};
}  // namespace

cudaError_t program_create(const std::vector<ProgEntry>& entries_in, const std::vector<int>& phase_of,
                           int sm_count, bool strict_phases, const ShardInfo* shard, Program** out, std::string* msg) {
  Program* p = new (std::nothrow) Program();
  if (!p) return cudaErrorMemoryAllocation;
  std::vector<ProgEntry> entries = entries_in;
  std::vector<ProgPhase> phases;
  std::vector<CUtensorMap> maps(entries.size());
  std::vector<Produced> made(entries.size());
  std::vector<int> phase_idx(entries.size());
  const int world = shard ? shard->world : 1, rank = shard ? shard->rank : 0;
  size_t tagged_bytes = 0;
  auto fail = [&](const char* m, cudaError_t e) {
    if (msg) *msg = m;
    delete p;
    return e;
  };
  // sharded: the tagged pair of the float at arena address a
  auto arena_tagged = [&](const char* a) -> char* {
    const char* res0 = shard->arena + LLR_ARENA_HEADER_BYTES_INTERNAL;
    return shard->arena + LLR_ARENA_HEADER_BYTES_INTERNAL + shard->result_bytes + 2 * (a - res0);
  };
  for (size_t i = 0; i < entries.size(); ++i) {
    ProgEntry& E = entries[i];
    if (!encode_weight_map(E.w, E.dtype, E.rows, E.cols, E.row_bytes, &maps[i]))
      return fail("tensor map of an entry could not be encoded", cudaErrorNotSupported);
    E.n_tiles = (E.rows + 15) / 16;
    if (E.y_ld == 0) E.y_ld = E.rows;
    if (i == 0 || phase_of[i] != phase_of[i - 1]) phases.push_back(ProgPhase{(int)i, 0, 0, 0});
    ProgPhase& P = phases.back();
    const int ph = (int)phases.size() - 1;
    phase_idx[i] = ph;
    E.tile_begin = P.n_tiles;
    P.n_tiles += E.n_tiles;
    ++P.n_entries;
    if (E.tokens > p->max_tokens) p->max_tokens = E.tokens;
    const bool addressable = world == 1 || E.y_ld == (int64_t)world * E.rows;
    const int64_t row0 = world == 1 ? 0 : (int64_t)rank * E.rows;
    made[i] = Produced{(const char*)E.y - 4 * row0, E.y_ld, E.tokens, ph, SIZE_MAX, addressable, false};
    // Resolve each input: the latest earlier-phase result that contains it becomes a tagged source.
    // width floats per activation row are read starting at ptr.
    auto resolve = [&](const void* ptr, int64_t width, int* src_phase) -> const void* {
      *src_phase = -1;
      if (!ptr) return nullptr;
      if (strict_phases) return ptr;  // strict programs synchronise phase by phase; their results travel as plain floats
      for (size_t j = i; j-- > 0;) {
        Produced& Q = made[j];
        if (Q.phase >= ph || !Q.addressable || Q.tokens != E.tokens) continue;
        const char* c = (const char*)ptr;
        const bool whole = c == Q.base && width == Q.ld;
        const bool part = E.tokens == 1 && c >= Q.base && c + 4 * width <= Q.base + 4 * Q.ld && (c - Q.base) % 16 == 0;
        if (!whole && !part) continue;
        *src_phase = Q.phase;
        Q.consumed = true;
        if (shard) return arena_tagged(c);
        if (Q.tagged_off == SIZE_MAX) {
          Q.tagged_off = tagged_bytes;
          tagged_bytes += ((size_t)Q.tokens * (size_t)Q.ld * 8 + 255) & ~(size_t)255;
        }
        return (const void*)(uintptr_t)(Q.tagged_off + 2 * (size_t)(c - Q.base) + 1);  // offset + 1, rebased below
      }
      return ptr;
    };
    bool unresolved = false;
    int sp = -1;
    const void* r = resolve(E.x, E.cols, &sp);
    E.x_phase = sp;
    E.xt = sp >= 0 ? r : nullptr;
    unresolved = unresolved || sp < 0;
    if (E.x_op == XOP_SWIGLU) {
      if (!E.x2) return fail("a SwiGLU entry needs its second input", cudaErrorInvalidValue);
      E.x2 = resolve(E.x2, E.cols, &sp);
      E.x2_phase = sp;
      unresolved = unresolved || sp < 0;
    } else {
      E.x2_phase = -1;
    }
    if (E.resid) {
      const void* rr = resolve(E.resid, E.y_ld, &sp);
      E.resid_phase = sp;
      // indexed like y: this rank's slice
      if (sp >= 0) E.resid = shard ? (const void*)((const char*)rr + 8 * row0) : (const void*)((uintptr_t)rr + 8 * (size_t)row0);
      else E.resid = (const char*)E.resid + 4 * row0;
      unresolved = unresolved || sp < 0;
    } else {
      E.resid_phase = -1;
    }
    if (strict_phases && unresolved && ph > 0) P.wait_prev |= 1;
    if (E.x_phase >= 0 || E.x2_phase >= 0 || E.resid_phase >= 0 || E.x_op != XOP_NONE || E.resid) p->flow = true;
  }
  for (size_t k = 0; k < phases.size(); ++k) p->counter_phases += phases[k].wait_prev & 1;
  if (p->counter_phases > 0) {
    // a counter phase needs its predecessor's count, and a sharded run must not overtake its predecessor:
    // every phase publishes (the grid is the same in every phase, so the counts stay in step)
    for (size_t k = 0; k < phases.size(); ++k) phases[k].wait_prev |= 2;
    if (shard) phases[0].wait_prev |= 4;
  }
  p->n_phases = (int)phases.size();
  p->n_entries = (int)entries.size();
  cudaError_t e;
  const int mt = p->max_tokens;
  const bool sharded = shard != nullptr;
#define LLR_PREP(MT) (p->flow ? prog_prepare<MT, true>(sm_count, &p->grid, sharded) : prog_prepare<MT, false>(sm_count, &p->grid, sharded))
  if (mt == 1) e = LLR_PREP(1);
  else if (mt == 2) e = LLR_PREP(2);
  else if (mt <= 4) e = LLR_PREP(4);
  else e = LLR_PREP(8);
#undef LLR_PREP
  if (e == cudaSuccess && !sharded && tagged_bytes > 0) {
    e = cudaMalloc(&p->d_tagged, tagged_bytes);
    if (e == cudaSuccess) e = cudaMemset(p->d_tagged, 0, tagged_bytes);
  }
  // tagged addresses: single GPU offsets become pointers; producers learn where their tagged copy goes
  for (size_t i = 0; i < entries.size() && e == cudaSuccess; ++i) {
    ProgEntry& E = entries[i];
    if (!sharded) {
      auto rebase = [&](const void* v) { return (const void*)((char*)p->d_tagged + ((uintptr_t)v - 1)); };
      if (E.x_phase >= 0) E.xt = rebase(E.xt);
      if (E.x2_phase >= 0) E.x2 = rebase(E.x2);
      if (E.resid_phase >= 0) E.resid = rebase(E.resid);
      E.yt = made[i].tagged_off == SIZE_MAX ? nullptr : (char*)p->d_tagged + made[i].tagged_off;
    } else {
      // every rank creates the same program, so what is read here is read on the peers too
      E.yt = made[i].consumed ? (void*)arena_tagged((const char*)E.y) : nullptr;
    }
  }
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->d_entries, entries.size() * sizeof(ProgEntry));
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->d_phases, phases.size() * sizeof(ProgPhase));
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->d_maps, maps.size() * sizeof(CUtensorMap));
  if (e == cudaSuccess) e = cudaMemcpy(p->d_maps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
  if (sharded) {
    p->own_counters = false;
    p->d_counters = shard->counters;  // zeroed by whoever allocated the arena, before any rank runs
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->d_peers, sizeof(PeerTable));
    if (e == cudaSuccess) e = cudaMemcpy(p->d_peers, &shard->peers, sizeof(PeerTable), cudaMemcpyHostToDevice);
    // An arena that served an earlier program carries that program's counts and tags: the tags go on
    // from where it stopped and the counters start from zero again, so that neither a stale tag nor a
    // stale count can pass for a new one.  (No rank may still be running a program on these arenas.)
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(&p->tag_next, shard->counters + TAG_SLOT, sizeof(p->tag_next), cudaMemcpyDeviceToHost);
    if (p->tag_next == 0) p->tag_next = 1;
    if (e == cudaSuccess) e = cudaMemset(shard->counters, 0, TAG_SLOT * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(shard->counters + PEER_COUNTER_OFFSET, 0, (COUNTER_WORDS - PEER_COUNTER_OFFSET) * sizeof(unsigned long long));
  } else {
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->d_counters, COUNTER_WORDS * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(p->d_counters, 0, COUNTER_WORDS * sizeof(unsigned long long));
  }
  if (e == cudaSuccess) e = cudaMemcpy(p->d_entries, entries.data(), entries.size() * sizeof(ProgEntry), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(p->d_phases, phases.data(), phases.size() * sizeof(ProgPhase), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    if (msg) *msg = cudaGetErrorString(e);
    program_destroy(p);
    return e;
  }
  *out = p;
  return cudaSuccess;
}

cudaError_t program_set_select(Program* p, const void* maps_dev, const int* sel_dev) {
  if (p->n_phases != 1 || p->counter_phases != 0 || p->flow || p->max_tokens != 1 || p->d_peers) return cudaErrorInvalidValue;
  int bps = 0;  // the grid stays the plain program's: no CTA waits for another, so residency does not matter
  cudaError_t e = occupancy(gemv_select_program_kernel, SLay<1>::TOTAL, &bps);
  if (e != cudaSuccess) return e;
  p->sel_maps = (const CUtensorMap*)maps_dev;
  p->sel = sel_dev;
  return cudaSuccess;
}

void program_destroy(Program* p) {
  if (!p) return;
  if (p->d_entries) cudaFree(p->d_entries);
  if (p->d_phases) cudaFree(p->d_phases);
  if (p->d_maps) cudaFree(p->d_maps);
  if (p->d_counters && p->own_counters) cudaFree(p->d_counters);
  if (p->d_tagged) cudaFree(p->d_tagged);
  if (p->d_peers) cudaFree(p->d_peers);
  delete p;
}

cudaError_t program_run(Program* p, cudaStream_t stream, int* err_flag, int poll_limit, uint64_t* launches) {
  cudaError_t e;
  const int mt = p->max_tokens;
#define LLR_RUN(MT) (p->flow ? prog_launch<MT, true>(p, stream, err_flag, poll_limit) : prog_launch<MT, false>(p, stream, err_flag, poll_limit))
  if (mt == 1) e = LLR_RUN(1);
  else if (mt == 2) e = LLR_RUN(2);
  else if (mt <= 4) e = LLR_RUN(4);
  else e = LLR_RUN(8);
#undef LLR_RUN
  if (e == cudaSuccess && launches) ++*launches;
  return e;
}

int program_counter_phases(const Program* p) { return p->counter_phases; }
int program_grid(const Program* p) { return p->grid; }
int program_phases(const Program* p) { return p->n_phases; }
int program_entries(const Program* p) { return p->n_entries; }

}  // namespace llr
