// Launch-shape knobs.  Each has a built-in default chosen from measurements on B200; a value set
// through mxk_set_tuning() overrides it process-wide (0 restores the default).  They change how
// the work is tiled, never the results.
#pragma once

namespace mxk {

enum TuneKey {
  TUNE_NORM_THREADS = 0,   // preferred CTA size of the row-norm kernels
  TUNE_NORM_CTAS_PER_SM,   // CTAs per SM the row-norm grid is sized for (unset: one resident wave; the residual-only mode: one row per CTA)
  TUNE_ROPE_THREADS,       // CTA size of head_norm_rope
  TUNE_ROPE_CTAS_PER_SM,
  TUNE_RES_ROWS_PER_CTA,   // rows each gated_residual CTA walks
  TUNE_RES_THREADS,
  TUNE_EW_THREADS,         // CTA size of the flat elementwise kernels
  TUNE_EW_UNROLL,          // independent 16-byte vectors per thread (1, 2, 4 or 8)
  TUNE_ACT_ROWS_PER_CTA,   // rows each silu_mul CTA walks
  TUNE_NORM_PATH,          // 1 bulk-copy (TMA) pipelined row kernel, 2 register-prefetch row kernel
  TUNE_NORM_STAGES,        // rows in flight per CTA of the bulk-copy kernel (2..8)
  TUNE_ROPE_PATH,          // 1 bulk-copy (TMA) pipelined head kernel (default), 2 register head kernel, 3 D = 128: one group of tokens per CTA straight from global memory
  TUNE_ROPE_STAGES,        // tokens in flight per CTA of the bulk-copy head kernel (2..8)
  TUNE_EW_CTAS_PER_SM,     // CTAs per SM the flat elementwise grid is capped at (unset: no cap, one tile per CTA)
  TUNE_RES_PATH,           // 1 bulk-copy pipelined gated_residual, 2 column-strip register kernel
  TUNE_ROPE_TOKENS,        // tokens per stage of the bulk-copy head kernel (1..16)
  TUNE_STREAM_WARPS,       // consumer warps per CTA of the streaming pipeline
  TUNE_STREAM_STAGES,      // its stages (2..8)
  TUNE_STREAM_CTAS_PER_SM,
  TUNE_STREAM_CHUNK_KB,    // bytes per source per chunk, in KB
  TUNE_ACT_PATH,           // activations: 1 bulk-copy streaming pipeline, 2 register kernels on one resident wave (GELU: the flat kernel, one tile per CTA), 3 silu_mul with one tile per CTA; unset: GELU 2, silu_mul 3
  TUNE_PDL,                // 2 disables programmatic dependent launch (default: on)
  TUNE_NORM_INTERLEAVE,    // 1: CTA i of the bulk-copy row kernels takes rows i, i + grid, ...; 2: contiguous ranges
  TUNE_PIPE_INTERLEAVE,    // same choice for the head and streaming pipelines (1 interleaved, 2 contiguous)
  TUNE_QUANT_ROWS_PER_CTA, // rows per work item of the block-scale quantiser
  TUNE_QUANT_PATH,         // 1 bulk-copy streaming pipeline, 2 register kernels on one resident wave, 3 a thread per scale block (NVFP4: per pair) and a row per CTA; unset: MXFP8 3, NVFP4 1
  TUNE_ROPE_UNROLL,        // 1: head pipeline with the pass loop unrolled where the shape allows (default), 2: runtime loop
  TUNE_ROPE_WIDE,          // 1: sixteen channels per lane for D = 128, 2: eight channels per lane (default)
  TUNE_ROPE_WIDE_REGS,     // wide head kernel's register budget: 1 = 128 registers for CTAs of up to 128 threads (default), 2 = 96 everywhere
  TUNE_LINEAR_CTAS,        // linear layers: 2 = a pair of CTAs per 256 x 256 tile, 1 = one CTA per 128 x 256 tile, 0 = whichever needs fewer waves (default)
  TUNE_LINEAR_GROUP_M,     // linear layers: row tiles per band of the tile order (default 8 for CTA pairs, 16 for single CTAs)
  TUNE_COUNT
};

int tune(int key, int dflt);

}  // namespace mxk
