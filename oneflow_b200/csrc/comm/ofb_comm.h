// C ABI of the communication part of libofb_kernels.so (symmetric memory, stand-alone collectives,
// GEMM fused with reduce-scatter / all-gather). Bound from Python in oneflow_b200/comm/symmetric.py.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct OfbCommCtx {
  int rank;
  int n;
  void* arena[8];    // arena base of every rank as mapped into this process
  void* signals[8];  // SignalBlock of every rank as mapped into this process
} OfbCommCtx;

// One rank's shard of an embedding: open-addressing key index (power-of-two `tcap`, empty = all ones) over
// densely allocated fp32 rows of `line` floats ([weights (dim) | optimizer state]).
// One slot of the key index: everything a lookup needs sits in one 32-byte sector.
typedef struct OfbEmbSlot {
  unsigned long long key;       // all ones = empty
  int row;                      // row of the key (-1: none)
  int uo;                       // number of the key among the rows touched in the step `stamp`
  unsigned int stamp;           // last step that touched the key
  int pad[3];
} OfbEmbSlot;

typedef struct OfbEmbStore {
  OfbEmbSlot* slots;            // [tcap]
  float* rows;                  // [row_cap][line]
  unsigned long long* row_key;  // [row_cap] key of each row (snapshots)
  int* counters;                // [0] rows in use
  const int* init_kind;         // per table: 0 uniform(a, b), 1 normal(mean a, std b), 2 constant a
  const float* init_a;
  const float* init_b;
  long long tcap;
  long long row_cap;
  int line;
  int dim;
  int num_tables;
  float state_init;             // initial value of the optimizer-state part of a new row
  unsigned long long seed;
} OfbEmbStore;

// Exchange buffers of one embedding. The *_off regions live in the symmetric arena at the same offset on every
// rank; the pointers are this rank's private scratch.
typedef struct OfbEmbShuffle {
  long long keys_off;   // u64 [ranks][cap]      unique keys received from each rank
  long long cnt_off;    // i32 [2][8]            their counts, double-buffered by step parity
  long long emb_off;    // 16-bit [ranks][cap][dim] rows received from each owner
  long long grad_off;   // 16-bit [ranks][cap][dim] gradient rows received from each rank
  long long cap;        // ids per (source, owner) pair: at least the ids of one rank per step
  unsigned long long* dkeys;  // [dcap] per-step dedupe table
  unsigned int* dval;         // [dcap] owner << 28 | index of the key
  long long dcap;
  int* cnt;             // [8] unique keys of this step per owner
  unsigned int* inv;    // [cap] owner << 28 | index for every id position
  float* gsum;          // [ranks * cap][dim] per-key gradient sums (zero between steps)
  int* slot_tmp;        // [ranks * cap] owner side, per received key: table slot
  int* rowidx;          // [ranks * cap] its row
  int* uoidx;           // [ranks * cap] its number among the rows touched this step
  int* u_row;           // [ranks * cap] row of each touched-row number
  float* gacc;          // [ranks * cap][dim] summed gradient of each touched row (zero between steps)
  int* n_uo;            // [1] rows touched this step
  int* done;            // [2] CTA completion counters
} OfbEmbShuffle;

typedef struct OfbEmbUpdate {
  int kind;             // 0 sgd, 1 momentum, 2 adam, 3 adagrad, 4 ftrl, 5 smart-decay adam (rows: [w | m | v | last step ...])
  float lr, lr_eff, scale, weight_decay, l2, momentum, beta1, beta2, eps, bias_corr1, bias_corr2, lr_power, lambda1, lambda2, beta;
  int step;             // 1-based number of this update (smart-decay adam)
} OfbEmbUpdate;

int ofb_emb_forward(const OfbCommCtx* ctx, const OfbEmbStore* st, const OfbEmbShuffle* sh, const long long* ids, const int* tids,
                    long long n, int columns, int insert, unsigned int epoch, void* out, int out_half, void* stream);
int ofb_emb_backward(const OfbCommCtx* ctx, const OfbEmbStore* st, const OfbEmbShuffle* sh, const void* grad, long long n, int grad_half,
                     unsigned int epoch, const OfbEmbUpdate* upd, void* stream);
int ofb_emb_find(const OfbEmbStore* st, const long long* keys, long long n, int insert, int* rows, void* stream);

int ofb_symm_alloc(long long bytes, void** ptr, unsigned char* handle64);
int ofb_symm_open(const unsigned char* handle64, void** ptr);
int ofb_symm_close(void* ptr);
int ofb_symm_free(void* ptr);
int ofb_comm_collective(const OfbCommCtx* ctx, int mode, long long in_off, long long stage_off, int in_dtype, void* out,
                        int out_dtype, long long count, float scale, unsigned int epoch, int ctas, void* stream);
int ofb_comm_all_to_all(const OfbCommCtx* ctx, long long in_off, int dtype, void* out, long long outer, long long I,
                        long long mid, long long J, long long inner, unsigned int epoch, int ctas, void* stream);

#ifdef __cplusplus
}
#endif
