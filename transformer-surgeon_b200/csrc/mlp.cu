// Gated MLP block: y = down(silu(gate(x)) * up(x)), the whole of
// transformersurgeon/blocks/mlp.py:171-185 (MLPGated.forward) behind one entry point.
//
// When the three layers are packed alike (same container bits, bf16, 9 <= M <= 64) the block runs as
// ONE persistent tcgen05 launch of up to four phases (linear_tcq.cu): [gate V | up V] -> [gate U,
// up U with SiLU(g) * u in the epilogue] -> [down V] -> [down U].  Otherwise it is composed from
// tsb200_linear and tsb200_swiglu calls.
#include "tc_common.cuh"

using namespace tsb;

namespace {
size_t align256(size_t v) { return (v + 255) / 256 * 256; }

bool fusable(const tsb200_linear_desc* g, const tsb200_linear_desc* u, const tsb200_linear_desc* d, int64_t M) {
  if (g->act_dtype != TSB200_BF16 || u->act_dtype != TSB200_BF16 || d->act_dtype != TSB200_BF16) return false;
  if (M < 1 || M > 64) return false;
  const int bits = g->u_bits;
  if (!(bits == 2 || bits == 4 || bits == 8)) return false;
  if (u->u_bits != bits || d->u_bits != bits) return false;
  if ((g->rank > 0) != (u->rank > 0) || g->rank != u->rank) return false;
  if (g->rank > 0 && (g->v_bits != bits || u->v_bits != bits)) return false;
  if (d->rank > 0 && d->v_bits != bits) return false;
  if (g->bias || u->bias) { /* biases are supported by the fused epilogue */ }
  const int64_t dims[] = {g->in_features, g->out_features, g->rank, d->rank, d->out_features};
  for (int64_t v : dims)
    if (v % 8) return false;
  // the gated phase keeps each tile's K range whole: it must fill the machine without a K split
  const int64_t tiles = (g->out_features + tc::BM - 1) / tc::BM;
  if (tiles < tc::kPlanSMs * 3 / 8) return false;
  return true;
}
}  // namespace

// Workspace layout: [region 0 | gate out | up out | act | h0 | h1 | h2].  Region 0 starts with the
// zero-between-calls header (status, grid barrier, split-K counters) and continues with scratch that
// needs no initialisation: split-K slices (fused path) or the body of the nested tsb200_linear
// workspace (composed path).  Keeping the header at offset 0 in both paths makes one workspace
// reusable across differently shaped blocks.
static size_t region0_bytes(const tsb200_linear_desc* gate, const tsb200_linear_desc* up, const tsb200_linear_desc* down,
                            int64_t M) {
  size_t scratch = 0;
  if (gate->rank > 0) scratch += phase_scratch_bytes(M, gate->rank, gate->in_features, 2, false);
  if (down->rank > 0) {
    scratch += phase_scratch_bytes(M, down->rank, down->in_features, 1, false);
    scratch += phase_scratch_bytes(M, down->out_features, down->rank, 1, false);
  } else {
    scratch += phase_scratch_bytes(M, down->out_features, down->in_features, 1, false);
  }
  size_t r0 = tc::kWsHeader + scratch;
  const size_t l1 = tsb200_linear_workspace_bytes(gate, M), l2 = tsb200_linear_workspace_bytes(up, M),
               l3 = tsb200_linear_workspace_bytes(down, M);
  if (l1 > r0) r0 = l1;
  if (l2 > r0) r0 = l2;
  if (l3 > r0) r0 = l3;
  return align256(r0);
}

extern "C" {

size_t tsb200_mlp_gated_workspace_bytes(const tsb200_linear_desc* gate, const tsb200_linear_desc* up,
                                        const tsb200_linear_desc* down, int64_t M) {
  if (!gate || !up || !down || M <= 0) return tc::kWsHeader;
  const size_t elt = gate->act_dtype == TSB200_F32 ? 4 : 2;
  size_t b = region0_bytes(gate, up, down, M);
  b += 3 * align256((size_t)M * (size_t)gate->out_features * elt);
  b += 3 * align256((size_t)M * (size_t)(gate->rank > down->rank ? gate->rank : down->rank) * elt);
  return b + 256;
}

int tsb200_mlp_gated(const tsb200_linear_desc* gate, const tsb200_linear_desc* up, const tsb200_linear_desc* down,
                     const void* x, void* y, int64_t M, void* workspace, size_t workspace_bytes, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (!gate || !up || !down || M < 0) return TSB200_ERR_ARG;
  if (gate->in_features != up->in_features || gate->out_features != up->out_features ||
      down->in_features != gate->out_features)
    return TSB200_ERR_ARG;
  if (gate->act_dtype != up->act_dtype || gate->act_dtype != down->act_dtype) return TSB200_ERR_ARG;
  if (M == 0) return TSB200_OK;
  if (!x || !y || !workspace || !aligned(workspace, 256)) return TSB200_ERR_ARG;
  if (workspace_bytes < tsb200_mlp_gated_workspace_bytes(gate, up, down, M)) return TSB200_ERR_WORKSPACE;
  cudaStream_t s = as_stream(stream);
  uint8_t* ws = (uint8_t*)workspace;
  const size_t elt = gate->act_dtype == TSB200_F32 ? 4 : 2;
  const size_t r0 = region0_bytes(gate, up, down, M);
  const size_t inter_b = align256((size_t)M * (size_t)gate->out_features * elt);
  const size_t r_b = align256((size_t)M * (size_t)(gate->rank > down->rank ? gate->rank : down->rank) * elt);
  uint8_t* buf_g = ws + r0;                     // gate out (composed path) / act (fused path)
  uint8_t* buf_u = buf_g + inter_b;
  uint8_t* buf_a = buf_u + inter_b;
  uint8_t* h0 = buf_a + inter_b;
  uint8_t* h1 = h0 + r_b;
  uint8_t* h2 = h1 + r_b;

  if (fusable(gate, up, down, M)) {
    PhaseSpec ps[4];
    int n = 0;
    const void* gx = x;
    const void* ux = x;
    if (gate->rank > 0) {
      ps[n].nsub = 2; ps[n].gated = 0;
      ps[n].g[0] = GemmSpec{gate->v, gate->v_scale, nullptr, x, h0, gate->rank, gate->in_features};
      ps[n].g[1] = GemmSpec{up->v, up->v_scale, nullptr, x, h1, up->rank, up->in_features};
      ++n;
      gx = h0;
      ux = h1;
    }
    const int64_t kgu = gate->rank > 0 ? gate->rank : gate->in_features;
    ps[n].nsub = 2; ps[n].gated = 1;
    ps[n].g[0] = GemmSpec{gate->u, gate->u_scale, gate->bias, gx, buf_g, gate->out_features, kgu};
    ps[n].g[1] = GemmSpec{up->u, up->u_scale, up->bias, ux, buf_g, up->out_features, kgu};
    ++n;
    if (down->rank > 0) {
      ps[n].nsub = 1; ps[n].gated = 0;
      ps[n].g[0] = GemmSpec{down->v, down->v_scale, nullptr, buf_g, h2, down->rank, down->in_features};
      ++n;
      ps[n].nsub = 1; ps[n].gated = 0;
      ps[n].g[0] = GemmSpec{down->u, down->u_scale, down->bias, h2, y, down->out_features, down->rank};
      ++n;
    } else {
      ps[n].nsub = 1; ps[n].gated = 0;
      ps[n].g[0] = GemmSpec{down->u, down->u_scale, down->bias, buf_g, y, down->out_features, down->in_features};
      ++n;
    }
    const int st = run_program_tcq(ps, n, gate->u_bits, M, ws + tc::kWsHeader, (int*)(ws + tc::kWsCounters),
                                   (int*)(ws + tc::kWsGridBar), (int*)ws, s);
    if (st != TSB200_ERR_UNSUPPORTED) return st;
  }
  // composed path: three linear calls and the SwiGLU kernel; region 0 is their workspace
  int st = tsb200_linear(gate, x, buf_g, M, ws, r0, stream);
  if (st != TSB200_OK) return st;
  st = tsb200_linear(up, x, buf_u, M, ws, r0, stream);
  if (st != TSB200_OK) return st;
  const int64_t inter = gate->out_features;
  st = tsb200_swiglu(buf_g, buf_u, buf_a, gate->act_dtype, M, inter, inter, inter, inter, stream);
  if (st != TSB200_OK) return st;
  return tsb200_linear(down, buf_a, y, M, ws, r0, stream);
}

}  // extern "C"
