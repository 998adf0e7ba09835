// MX block quantisation launchers (bf16 -> e4m3 + E8M0 per 32) and scale-factor re-layout.
#pragma once
#include "symm_heap.h"

namespace cb {

// Bytes of the tcgen05 scale-factor atom layout for a [rows, k] operand:
// atoms of 128 rows x 4 k-blocks (512 B), ordered [row tile][k / 128].
size_t sf_atoms_bytes(int rows, int k);

// codes[r, :] = e4m3(in[r, :] / 2^exp), one E8M0 scale per 32 along k.  scales_rm (optional):
// [rows, scale_ld] bytes, count padded to even with 127.  sf_atoms (optional): the same scales in
// the atom layout (pad positions 127).
int mx_quant_launch(cudaStream_t stream, const void *in_bf16, int rows, int k, uint8_t *codes, size_t code_ld,
                    uint8_t *scales_rm, int scale_ld, uint8_t *sf_atoms);

// kind 0: src [rows, ld];  kind 1: src [kblocks/2, rows, 2]
int sf_to_atoms_launch(cudaStream_t stream, const uint8_t *src, int kind, int rows, int kblocks, int ld, uint8_t *atoms);

}  // namespace cb
