// Static work plan of the persistent decode kernel (decoder_persistent.cu): which cells of which
// weight matrix every CTA streams in every phase of a layer, cut into the bulk copies ("chunks")
// that travel through the CTA's shared-memory ring.  Host code only; the plan depends on the model
// shape and the CTA count, not on the weights, and is the same for every layer.
//
// Phases with weights (one decoder layer):
//   0  q,k,v   cell space = panels of q, then k, then v (x their K-groups), cut evenly over the CTAs
//   1  o       cut evenly
//   2  gate,up whole panel pairs (gate panel p + up panel p on the same CTA: it finishes silu(g)*u)
//   3  down    cut evenly
// A CTA's share of a phase is a run of cells; the part of a run inside one panel is a "panel run".
// Panel runs that do not cover all K-groups of their panel produce partial sums: the panel run of
// the i-th CTA that touches a panel writes slot i, and the consumer adds the slots in order.
#pragma once
#include <stdint.h>

#include <vector>

#include "layout.h"

namespace mllmb200 {

constexpr int kPlanChunkCells = 16;  // cells per bulk copy (16 * 576 = 9216 bytes)
constexpr int kPlanMaxSlots = 8;     // partial-sum slots per output row
constexpr int kPlanPhases = 4;

enum : uint8_t { kChunkFirstOfRun = 1, kChunkLastOfRun = 2 };

struct PlanChunk {       // 16 bytes
  uint32_t byte_off;     // from the start of the linear's tiled buffer
  uint16_t ncells;       // 1 .. kPlanChunkCells
  uint8_t lin;           // 0 q, 1 k, 2 v, 3 o, 4 gate, 5 up, 6 down
  uint8_t flags;         // kChunkFirstOfRun | kChunkLastOfRun
  uint16_t panel;        // panel inside its linear
  uint16_t group0;       // first K-group of the chunk
  uint16_t slot;         // partial-sum slot of the panel run
  uint16_t run_groups;   // K-groups of the whole panel run (== all groups of the panel: complete sums)
};
static_assert(sizeof(PlanChunk) == 16, "PlanChunk is 16 bytes");

struct DecodePlan {
  int nctas = 0, max_chunks = 0;             // chunks per CTA per layer, padded to max_chunks
  std::vector<PlanChunk> chunks;             // [ncta][max_chunks]
  std::vector<int> phase_begin;              // [ncta][kPlanPhases + 1] chunk index ranges per phase
  std::vector<uint8_t> slots_qkv, slots_o, slots_down;  // slots per panel (qkv: concatenated panels)
  int max_slots = 0;
};

struct PlanShape {
  int hidden, q_dim, kv_dim, inter;  // all multiples of 32
};

namespace plan_detail {
struct Lin {
  int lin, panels, groups;
};
// Appends the chunks of cells [c0, c1) of the concatenated cell space of `lins` to `out`.
inline void emit_run(const Lin* lins, int nl, long c0, long c1, std::vector<PlanChunk>& out,
                     std::vector<std::vector<uint8_t>*> slot_tables, const int* cat_panel_base) {
  long base = 0;
  for (int i = 0; i < nl && c0 < c1; ++i) {
    const long cells = (long)lins[i].panels * lins[i].groups;
    const long lo = c0 > base ? c0 : base, hi = c1 < base + cells ? c1 : base + cells;
    for (long c = lo; c < hi;) {
      const int panel = (int)((c - base) / lins[i].groups), g0 = (int)((c - base) % lins[i].groups);
      const long run_end = (hi - base) < (long)(panel + 1) * lins[i].groups ? hi : base + (long)(panel + 1) * lins[i].groups;
      const int run_groups = (int)(run_end - c);
      std::vector<uint8_t>& tab = *slot_tables[i];
      const int slot = tab[cat_panel_base[i] + panel]++;
      for (int g = g0; g < g0 + run_groups; g += kPlanChunkCells) {
        PlanChunk ch{};
        ch.ncells = (uint16_t)((g0 + run_groups - g) < kPlanChunkCells ? (g0 + run_groups - g) : kPlanChunkCells);
        ch.lin = (uint8_t)lins[i].lin;
        ch.panel = (uint16_t)panel;
        ch.group0 = (uint16_t)g;
        ch.slot = (uint16_t)slot;
        ch.run_groups = (uint16_t)run_groups;
        ch.byte_off = (uint32_t)(sizeof(TiledHeader) + ((size_t)panel * lins[i].groups + g) * kCellBytes);
        ch.flags = (uint8_t)((g == g0 ? kChunkFirstOfRun : 0) | (g + kPlanChunkCells >= g0 + run_groups ? kChunkLastOfRun : 0));
        out.push_back(ch);
      }
      c = run_end;
    }
    base += cells;
  }
}
}  // namespace plan_detail

// Returns false when the shape cannot be planned (too many partial slots, offsets out of range).
inline bool build_decode_plan(const PlanShape& s, int nctas, DecodePlan* plan) {
  using namespace plan_detail;
  if (nctas < 1 || (s.hidden % 32) || (s.q_dim % 32) || (s.kv_dim % 32) || (s.inter % 32)) return false;
  const int gh = s.hidden / 32, gq = s.q_dim / 32, gi = s.inter / 32;
  const Lin qkv[3] = {{0, s.q_dim / 32, gh}, {1, s.kv_dim / 32, gh}, {2, s.kv_dim / 32, gh}};
  const Lin o[1] = {{3, s.hidden / 32, gq}};
  const Lin down[1] = {{6, s.hidden / 32, gi}};
  const int qkv_base[3] = {0, s.q_dim / 32, s.q_dim / 32 + s.kv_dim / 32};
  const int zero_base[1] = {0};
  plan->nctas = nctas;
  plan->slots_qkv.assign(s.q_dim / 32 + 2 * (s.kv_dim / 32), 0);
  plan->slots_o.assign(s.hidden / 32, 0);
  plan->slots_down.assign(s.hidden / 32, 0);
  std::vector<uint8_t> slots_gate(s.inter / 32, 0), slots_up(s.inter / 32, 0);
  std::vector<std::vector<PlanChunk>> per_cta(nctas);
  plan->phase_begin.assign((size_t)nctas * (kPlanPhases + 1), 0);
  const long t_qkv = (long)(s.q_dim / 32 + 2 * (s.kv_dim / 32)) * gh, t_o = (long)(s.hidden / 32) * gq,
             t_down = (long)(s.hidden / 32) * gi;
  const int pairs = s.inter / 32;
  // A run of at least ceil(G / (slots - 1)) cells keeps a panel of G groups within `slots` CTAs;
  // small matrices therefore use fewer CTAs.
  auto active_ctas = [&](long total, int groups) {
    const long min_run = (groups + kPlanMaxSlots - 2) / (kPlanMaxSlots - 1);
    const long a = total / min_run;
    return (int)(a < 1 ? 1 : (a < nctas ? a : nctas));
  };
  const int a_qkv = active_ctas(t_qkv, gh), a_o = active_ctas(t_o, gq), a_down = active_ctas(t_down, gi);
  auto cut = [](long total, int c, int active) { return c >= active ? total : total * c / active; };
  for (int c = 0; c < nctas; ++c) {
    std::vector<PlanChunk>& out = per_cta[c];
    int* pb = &plan->phase_begin[(size_t)c * (kPlanPhases + 1)];
    pb[0] = 0;
    emit_run(qkv, 3, cut(t_qkv, c, a_qkv), cut(t_qkv, c + 1, a_qkv), out, {&plan->slots_qkv, &plan->slots_qkv, &plan->slots_qkv},
             qkv_base);
    pb[1] = (int)out.size();
    emit_run(o, 1, cut(t_o, c, a_o), cut(t_o, c + 1, a_o), out, {&plan->slots_o}, zero_base);
    pb[2] = (int)out.size();
    for (int p = (int)((long)pairs * c / nctas); p < (int)((long)pairs * (c + 1) / nctas); ++p) {
      const Lin g[1] = {{4, pairs, gh}}, u[1] = {{5, pairs, gh}};
      emit_run(g, 1, (long)p * gh, (long)(p + 1) * gh, out, {&slots_gate}, zero_base);
      emit_run(u, 1, (long)p * gh, (long)(p + 1) * gh, out, {&slots_up}, zero_base);
    }
    pb[3] = (int)out.size();
    emit_run(down, 1, cut(t_down, c, a_down), cut(t_down, c + 1, a_down), out, {&plan->slots_down}, zero_base);
    pb[4] = (int)out.size();
    if ((int)out.size() > plan->max_chunks) plan->max_chunks = (int)out.size();
  }
  plan->max_slots = 0;
  for (auto* t : {&plan->slots_qkv, &plan->slots_o, &plan->slots_down})
    for (uint8_t v : *t) plan->max_slots = v > plan->max_slots ? v : plan->max_slots;
  if (plan->max_slots > kPlanMaxSlots || plan->max_chunks == 0) return false;
  // the largest tiled buffer must be addressable by the 32-bit chunk offsets
  const size_t biggest = sizeof(TiledHeader) + (size_t)pairs * gh * kCellBytes;
  const size_t biggest2 = sizeof(TiledHeader) + (size_t)(s.hidden / 32) * gi * kCellBytes;
  if (biggest > 0xFFFFFFFFull || biggest2 > 0xFFFFFFFFull) return false;
  plan->chunks.assign((size_t)nctas * plan->max_chunks, PlanChunk{});
  for (int c = 0; c < nctas; ++c)
    for (size_t i = 0; i < per_cta[c].size(); ++i) plan->chunks[(size_t)c * plan->max_chunks + i] = per_cta[c][i];
  return true;
}

// Self-check used by the tests: every cell of every linear is covered exactly once, runs do not
// cross panels, gate/up panels are complete and paired, slot numbering is dense.  Returns 0 when
// the plan is consistent, otherwise a positive code naming the failed check.
inline int check_decode_plan(const PlanShape& s, const DecodePlan& p) {
  const int panels[7] = {s.q_dim / 32, s.kv_dim / 32, s.kv_dim / 32, s.hidden / 32, s.inter / 32, s.inter / 32, s.hidden / 32};
  const int groups[7] = {s.hidden / 32, s.hidden / 32, s.hidden / 32, s.q_dim / 32, s.hidden / 32, s.hidden / 32, s.inter / 32};
  const int phase_of[7] = {0, 0, 0, 1, 2, 2, 3};
  std::vector<std::vector<uint8_t>> seen(7);
  for (int l = 0; l < 7; ++l) seen[l].assign((size_t)panels[l] * groups[l], 0);
  for (int c = 0; c < p.nctas; ++c) {
    const int* pb = &p.phase_begin[(size_t)c * (kPlanPhases + 1)];
    for (int ph = 0; ph < kPlanPhases; ++ph) {
      for (int i = pb[ph]; i < pb[ph + 1]; ++i) {
        const PlanChunk& ch = p.chunks[(size_t)c * p.max_chunks + i];
        if (ch.lin > 6 || phase_of[ch.lin] != ph) return 1;
        if (ch.ncells < 1 || ch.ncells > kPlanChunkCells) return 2;
        if (ch.panel >= panels[ch.lin] || ch.group0 + ch.ncells > groups[ch.lin]) return 3;
        if (ch.byte_off != sizeof(TiledHeader) + ((size_t)ch.panel * groups[ch.lin] + ch.group0) * kCellBytes) return 4;
        if ((ch.lin == 4 || ch.lin == 5) && ch.run_groups != groups[ch.lin]) return 5;
        if (ch.slot >= kPlanMaxSlots) return 6;
        for (int g = 0; g < ch.ncells; ++g) {
          uint8_t& v = seen[ch.lin][(size_t)ch.panel * groups[ch.lin] + ch.group0 + g];
          if (v) return 7;
          v = 1;
        }
        // gate panel p is followed (inside the same CTA) by up panel p
        if (ch.lin == 4 && (ch.flags & kChunkLastOfRun)) {
          if (i + 1 >= pb[ph + 1]) return 8;
          const PlanChunk& nx = p.chunks[(size_t)c * p.max_chunks + i + 1];
          if (nx.lin != 5 || nx.panel != ch.panel || !(nx.flags & kChunkFirstOfRun)) return 8;
        }
      }
    }
  }
  for (int l = 0; l < 7; ++l)
    for (uint8_t v : seen[l])
      if (!v) return 9;
  return 0;
}

}  // namespace mllmb200
