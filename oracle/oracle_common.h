/*
 * CPU oracle for the entropack compression hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * Plain-C restatement of the reference's eager (numpy/torch CPU) lanes. Nothing in the shipped
 * package links, imports or executes this code: it is used by the test suite, by the smoke check
 * and by the CPU-baseline leg of the benchmark, always as the checker and never as the product.
 *
 * Parity status: the reference ships no golden vectors, so this oracle is pinned against outputs of
 * the reference's own eager lanes run on seeded inputs (fixtures under tests/golden/, written by
 * tests/golden/make_golden.py). DFloat11 codeword assignment is delegated by the reference to a
 * third-party Huffman package that is not available; that one choice is "parity unpinned" (any
 * prefix code is decodable by the reference because the bitstream carries its own tables).
 */
#ifndef ENTROPACK_ORACLE_COMMON_H
#define ENTROPACK_ORACLE_COMMON_H

#include <stdint.h>
#include <stddef.h>

#define ORC_NUM_STATES 32
#define ORC_STATE_MIN (1u << 15)

#define ORC_OK 0
#define ORC_ERR_ARG (-1)
#define ORC_ERR_NORMALIZE (-2)
#define ORC_ERR_TRUNCATED (-3)
#define ORC_ERR_UNREAD (-4)
#define ORC_ERR_RAW_LENGTH (-5)
#define ORC_ERR_ALLOC (-6)
#define ORC_ERR_ALPHABET (-7)

#ifdef __cplusplus
extern "C" {
#endif

/* Largest-remainder normalisation of a histogram to `table_size`, present symbols >= 1, ties to the
 * smaller symbol index. Heap formulation: entropack/schemes/tile_ans/eager.py:16-48. The sorted
 * multi-pass formulation of entropack/schemes/lattice_rans/rans.py:12-53 gives the same result. */
int orc_normalize_counts(const int64_t* counts, int n, int table_size, uint16_t* freq_out);

/* sum c * (pb - log2 f) over present symbols: tile_ans/eager.py:81-85, lattice_rans/rans.py:56-59 */
double orc_quantized_cross_entropy(const int64_t* counts, const uint16_t* freq, int n, int prob_bits);

#ifdef __cplusplus
}
#endif

#endif
