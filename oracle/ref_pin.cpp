// Oracle pin: compiles two headers of the reference, unmodified and from where they lie, into a
// small host library so that the C restatement in ivfpq_oracle.c can be checked against the
// reference's own code for
//   - the custom 8-bit float    (cpp/src/neighbors/ivf_pq/ivf_pq_fp_8bit.cuh)
//   - the bit-field code layout (cpp/src/neighbors/ivf_pq/ivf_pq_codepacking.cuh:
//     bitfield_view_t, write_vector_interleaved, run_on_vector)
// The headers are device code; here `__device__` is empty and `threadIdx` is a host object, so the
// same statements run on the CPU.  Everything they include from un-vendored libraries is replaced
// by the shims in ref_shims/.  TEST INFRASTRUCTURE ONLY; built into oracle/_ref/ by the Makefile.
#include <cstdint>
#include <cstring>
#include <cmath>
#include <cstdlib>
#include <algorithm>
#include <cuda_fp16.h>

#ifndef __device__
#define __device__
#endif
struct fake_tid { unsigned x = 0, y = 0, z = 0; };
static fake_tid threadIdx;
static fake_tid blockIdx;
static fake_tid blockDim;

#include "ivf_pq_fp_8bit.cuh"
#include "ivf_pq_codepacking.cuh"

using namespace cuvs::neighbors::ivf_pq;
using namespace cuvs::neighbors::ivf_pq::detail;

extern "C" {

uint8_t ref_fp8_encode(float v, int is_signed)
{
  return is_signed ? fp_8bit<5, true>(v).bitstring : fp_8bit<5, false>(v).bitstring;
}
float ref_fp8_decode(uint8_t b, int is_signed)
{
  return is_signed ? float(fp_8bit<5, true>(b)) : float(fp_8bit<5, false>(b));
}
uint16_t ref_fp8_decode_half(uint8_t b, int is_signed)
{
  half h = is_signed ? half(fp_8bit<5, true>(b)) : half(fp_8bit<5, false>(b));
  uint16_t u;
  std::memcpy(&u, &h, 2);
  return u;
}

}  // extern "C"

using extents_t = list_spec_interleaved<uint32_t, uint32_t>::list_extents;

template <uint32_t Bits>
static void pack_t(const uint8_t* codes, uint32_t n_rows, uint32_t pq_dim, uint32_t first, uint8_t* list,
                   uint32_t n_groups, uint32_t n_pieces)
{
  raft::device_mdspan<uint8_t, extents_t, raft::row_major> view(list, extents_t{n_groups, n_pieces});
  for (uint32_t i = 0; i < n_rows; i++) {
    write_vector_interleaved<Bits, 1>(view, first + i, i, pq_dim, [&](uint32_t in_ix, uint32_t j) {
      return codes[size_t(in_ix) * pq_dim + j];
    });
  }
}
template <uint32_t Bits>
static void unpack_t(const uint8_t* list, uint32_t n_rows, uint32_t pq_dim, uint32_t first,
                     uint8_t* codes, uint32_t n_groups, uint32_t n_pieces)
{
  raft::device_mdspan<const uint8_t, extents_t, raft::row_major> view(list,
                                                                     extents_t{n_groups, n_pieces});
  for (uint32_t i = 0; i < n_rows; i++) {
    run_on_vector<Bits>(view, first + i, i, pq_dim, [&](uint8_t code, uint32_t out_ix, uint32_t j) {
      codes[size_t(out_ix) * pq_dim + j] = code;
    });
  }
}

extern "C" {

// `list` holds n_groups * n_pieces * 512 bytes, n_pieces = ceil(pq_dim / (128 / bits)).
int ref_pack_list(const uint8_t* codes, uint32_t n_rows, uint32_t pq_dim, uint32_t bits, uint32_t first,
                  uint8_t* list, uint32_t n_groups)
{
  uint32_t np = (pq_dim + 128 / bits - 1) / (128 / bits);
  switch (bits) {
    case 4: pack_t<4>(codes, n_rows, pq_dim, first, list, n_groups, np); break;
    case 5: pack_t<5>(codes, n_rows, pq_dim, first, list, n_groups, np); break;
    case 6: pack_t<6>(codes, n_rows, pq_dim, first, list, n_groups, np); break;
    case 7: pack_t<7>(codes, n_rows, pq_dim, first, list, n_groups, np); break;
    case 8: pack_t<8>(codes, n_rows, pq_dim, first, list, n_groups, np); break;
    default: return -1;
  }
  return 0;
}
int ref_unpack_list(const uint8_t* list, uint32_t n_rows, uint32_t pq_dim, uint32_t bits, uint32_t first,
                    uint8_t* codes, uint32_t n_groups)
{
  uint32_t np = (pq_dim + 128 / bits - 1) / (128 / bits);
  switch (bits) {
    case 4: unpack_t<4>(list, n_rows, pq_dim, first, codes, n_groups, np); break;
    case 5: unpack_t<5>(list, n_rows, pq_dim, first, codes, n_groups, np); break;
    case 6: unpack_t<6>(list, n_rows, pq_dim, first, codes, n_groups, np); break;
    case 7: unpack_t<7>(list, n_rows, pq_dim, first, codes, n_groups, np); break;
    case 8: unpack_t<8>(list, n_rows, pq_dim, first, codes, n_groups, np); break;
    default: return -1;
  }
  return 0;
}
}
