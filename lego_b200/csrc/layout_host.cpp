// Host-side layout services; see layout_host.h.
#include "layout_host.h"

#include <algorithm>
#include <cstring>

namespace lego {

namespace {

constexpr int64_t kMaxSize = (int64_t)1 << 62;

struct Piece {  // value = (idx[src] / div) % mod, radix = mod
  int32_t src;
  int64_t div;
  int64_t mod;
};

bool mul_ok(int64_t a, int64_t b, int64_t* out) {
  if (a <= 0 || b <= 0) return false;
  if (a > kMaxSize / b) return false;
  *out = a * b;
  return true;
}

// Re-cut a big-endian digit string at the prefix products of `dims`.  A cut
// that falls inside a digit of radix a*b splits it into (div*b, a) and (div, b);
// a cut that no split can realise makes the layout non-foldable.
bool recut(std::vector<Piece> s, const std::vector<int64_t>& dims,
           std::vector<std::vector<Piece>>* comps) {
  comps->assign(dims.size(), {});
  for (int k = (int)dims.size() - 1; k >= 0; --k) {
    int64_t need = dims[k];
    std::vector<Piece>& c = (*comps)[k];
    while (need > 1) {
      if (s.empty()) return false;
      Piece p = s.back();
      s.pop_back();
      if (p.mod <= need) {
        if (need % p.mod) return false;
        c.insert(c.begin(), p);
        need /= p.mod;
      } else {
        if (p.mod % need) return false;
        c.insert(c.begin(), Piece{p.src, p.div, need});
        s.push_back(Piece{p.src, p.div * need, p.mod / need});
        need = 1;
      }
    }
  }
  return s.empty();
}

uint32_t ceil_log2(uint64_t d) {
  uint32_t s = 0;
  while (((uint64_t)1 << s) < d) ++s;
  return s;
}

}  // namespace

FastDiv make_fastdiv(uint64_t d) {
  FastDiv f{};
  if (d == 0) d = 1;
  f.d = (uint32_t)d;
  const uint32_t s = ceil_log2(d);
  if (((uint64_t)1 << s) == d) {
    f.mul = 0;
    f.shr = s;
    return f;
  }
  // d is not a power of two, so 2^(s-1) < d < 2^s and the quotient below is < 2^32.
  const unsigned __int128 num = (unsigned __int128)1 << (31 + s);
  f.mul = (uint32_t)((num + d - 1) / d);
  f.shr = s - 1;
  return f;
}

int32_t check_layout(const lego_layout_t* L, int64_t* size_out) {
  if (!L) return LEGO_ERR_NULL;
  if (L->rank < 1 || L->rank > LEGO_MAX_RANK) return LEGO_ERR_RANK;
  if (L->n_stages < 0 || L->n_stages > LEGO_MAX_STAGES) return LEGO_ERR_RANK;
  int64_t size = 1;
  for (int k = 0; k < L->rank; ++k) {
    if (L->dims[k] < 1) return LEGO_ERR_DIM;
    if (!mul_ok(size, L->dims[k], &size)) return LEGO_ERR_OVERFLOW;
  }
  for (int s = 0; s < L->n_stages; ++s) {
    const lego_stage_t& st = L->stages[s];
    if (st.n_blocks < 1 || st.n_blocks > LEGO_MAX_BLOCKS) return LEGO_ERR_RANK;
    int64_t ssize = 1;
    int total_rank = 0;
    for (int b = 0; b < st.n_blocks; ++b) {
      const lego_block_t& bl = st.blocks[b];
      if (bl.rank < 1 || bl.rank > LEGO_MAX_RANK) return LEGO_ERR_RANK;
      total_rank += bl.rank;
      if (total_rank > LEGO_MAX_RANK) return LEGO_ERR_RANK;
      bool seen[LEGO_MAX_RANK] = {};
      for (int i = 0; i < bl.rank; ++i) {
        if (bl.dims[i] < 1) return LEGO_ERR_DIM;
        if (!mul_ok(ssize, bl.dims[i], &ssize)) return LEGO_ERR_OVERFLOW;
        const int p = bl.perm[i];
        if (bl.kind == LEGO_BLOCK_REGP) {
          if (p < 0 || p >= bl.rank || seen[p]) return LEGO_ERR_PERM;
          seen[p] = true;
        }
      }
      if (bl.kind == LEGO_BLOCK_REGP) continue;
      if (bl.kind == LEGO_BLOCK_ANTIDIAG) {
        if (bl.rank != 2 || bl.dims[0] != bl.dims[1]) return LEGO_ERR_DIM;
      } else if (bl.kind == LEGO_BLOCK_REVERSE) {
        if (bl.rank != 2) return LEGO_ERR_DIM;
      } else if (bl.kind == LEGO_BLOCK_LUT) {
        if (!bl.lut_apply || !bl.lut_inv) return LEGO_ERR_NULL;
        int64_t bsz = 1;
        for (int i = 0; i < bl.rank; ++i)
          if (!mul_ok(bsz, bl.dims[i], &bsz)) return LEGO_ERR_OVERFLOW;
        if (bsz > LEGO_MAX_LUT) return LEGO_ERR_SIZE;
      } else {
        return LEGO_ERR_UNSUPPORTED;
      }
    }
    if (ssize != size) return LEGO_ERR_NOT_BIJECTIVE;
  }
  if (size_out) *size_out = size;
  return LEGO_OK;
}

int32_t fold_layout(const lego_layout_t* L, std::vector<Digit>* digits) {
  int64_t size = 0;
  const int32_t st = check_layout(L, &size);
  if (st != LEGO_OK) return st;

  std::vector<Piece> s;
  for (int k = 0; k < L->rank; ++k)
    if (L->dims[k] > 1) s.push_back(Piece{k, 1, L->dims[k]});

  for (int si = L->n_stages - 1; si >= 0; --si) {
    const lego_stage_t& stg = L->stages[si];
    std::vector<int64_t> sdims;
    for (int b = 0; b < stg.n_blocks; ++b)
      for (int i = 0; i < stg.blocks[b].rank; ++i) sdims.push_back(stg.blocks[b].dims[i]);
    std::vector<std::vector<Piece>> comps;
    if (!recut(s, sdims, &comps)) return LEGO_ERR_UNSUPPORTED;
    std::vector<Piece> next;
    int at = 0;
    for (int b = 0; b < stg.n_blocks; ++b) {
      const lego_block_t& bl = stg.blocks[b];
      if (bl.kind != LEGO_BLOCK_REGP) return LEGO_ERR_UNSUPPORTED;
      for (int i = 0; i < bl.rank; ++i) {
        const std::vector<Piece>& c = comps[at + bl.perm[i]];
        next.insert(next.end(), c.begin(), c.end());
      }
      at += bl.rank;
    }
    s.swap(next);
  }

  // Merge neighbours that are one digit of the same source.
  std::vector<Piece> merged;
  for (const Piece& p : s) {
    if (!merged.empty()) {
      Piece& q = merged.back();
      if (q.src == p.src && q.div == p.div * p.mod) {
        q.div = p.div;
        q.mod *= p.mod;
        continue;
      }
    }
    merged.push_back(p);
  }
  if ((int)merged.size() > LEGO_MAX_TERMS) return LEGO_ERR_UNSUPPORTED;

  int64_t suffix[LEGO_MAX_RANK];
  int64_t acc = 1;
  for (int k = L->rank - 1; k >= 0; --k) {
    suffix[k] = acc;
    acc *= L->dims[k];
  }
  digits->clear();
  digits->resize(merged.size());
  int64_t stride = 1;
  for (int j = (int)merged.size() - 1; j >= 0; --j) {
    Digit& d = (*digits)[j];
    d.src = merged[j].src;
    d.div = merged[j].div;
    d.mod = merged[j].mod;
    d.pos = suffix[d.src] * d.div;
    d.stride = stride;
    stride *= d.mod;
  }
  return LEGO_OK;
}

int32_t build_staged(const lego_layout_t* L, StagedProgram* out) {
  const int32_t st = check_layout(L, nullptr);
  if (st != LEGO_OK) return st;
  std::memset(out, 0, sizeof(*out));
  out->rank = L->rank;
  out->n_stages = L->n_stages;
  for (int k = 0; k < L->rank; ++k) out->dims[k] = L->dims[k];
  for (int s = 0; s < L->n_stages; ++s) {
    const lego_stage_t& stg = L->stages[s];
    DevStage& d = out->stages[s];
    d.n_blocks = stg.n_blocks;
    int at = 0;
    for (int b = 0; b < stg.n_blocks; ++b) {
      const lego_block_t& bl = stg.blocks[b];
      d.blk_start[b] = (int8_t)at;
      d.blk_rank[b] = (int8_t)bl.rank;
      d.blk_kind[b] = (int8_t)bl.kind;
      d.lut_apply[b] = bl.kind == LEGO_BLOCK_LUT ? bl.lut_apply : nullptr;
      d.lut_inv[b] = bl.kind == LEGO_BLOCK_LUT ? bl.lut_inv : nullptr;
      for (int i = 0; i < bl.rank; ++i) {
        d.dims[at + i] = bl.dims[i];
        const int p = (bl.kind == LEGO_BLOCK_REGP) ? bl.perm[i] : i;
        d.gperm[at + i] = (int8_t)(at + p);
        d.pdims[at + i] = bl.dims[p];
      }
      at += bl.rank;
    }
    d.rank = at;
  }
  return LEGO_OK;
}

void set_term(DigitTerm* t, int src, int dst, int64_t a, int64_t m, int64_t b) {
  t->src = src;
  t->dst = dst;
  t->a64 = (uint64_t)a;
  t->m64 = (uint64_t)m;
  t->b = (uint64_t)b;
  t->a = make_fastdiv((uint64_t)a);
  t->m = make_fastdiv(m ? (uint64_t)m : 1);
  if (m == 0) t->m.d = 0;
}

static int32_t is_wide(int64_t size) { return size > ((int64_t)1 << 31) ? 1 : 0; }

void program_range(const std::vector<Digit>& dg, int64_t size, DigitProgram* p) {
  std::memset(p, 0, sizeof(*p));
  p->n_src = 1;
  p->n_dst = 1;
  p->wide = is_wide(size);
  // Merge digits adjacent both in the logical flat id and in the output.
  struct T { int64_t pos, mod, stride; };
  std::vector<T> ts;
  for (const Digit& d : dg) {
    if (!ts.empty()) {
      T& q = ts.back();
      if (q.pos == d.pos * d.mod && q.stride == d.stride * d.mod) {
        q.pos = d.pos;
        q.stride = d.stride;
        q.mod *= d.mod;
        continue;
      }
    }
    ts.push_back(T{d.pos, d.mod, d.stride});
  }
  for (const T& t : ts) {
    const bool top = (t.pos * t.mod == size);
    set_term(&p->t[p->n_terms++], 0, 0, t.pos, top ? 0 : t.mod, t.stride);
  }
}

void program_apply(const std::vector<Digit>& dg, int rank, int64_t size, DigitProgram* p) {
  std::memset(p, 0, sizeof(*p));
  p->n_src = rank;
  p->n_dst = 1;
  p->wide = is_wide(size);
  for (const Digit& d : dg) set_term(&p->t[p->n_terms++], d.src, 0, d.div, d.mod, d.stride);
}

void program_inv(const std::vector<Digit>& dg, int rank, int64_t size, DigitProgram* p) {
  std::memset(p, 0, sizeof(*p));
  p->n_src = 1;
  p->n_dst = rank;
  p->wide = is_wide(size);
  for (const Digit& d : dg) {
    const bool top = (d.stride * d.mod == size);
    set_term(&p->t[p->n_terms++], 0, d.src, d.stride, top ? 0 : d.mod, d.div);
  }
}

bool refine_pair(const std::vector<Digit>& a, const std::vector<Digit>& b, std::vector<PairDigit>* out) {
  std::vector<int64_t> cuts;
  for (const Digit& d : a) { cuts.push_back(d.pos); cuts.push_back(d.pos * d.mod); }
  for (const Digit& d : b) { cuts.push_back(d.pos); cuts.push_back(d.pos * d.mod); }
  std::sort(cuts.begin(), cuts.end());
  cuts.erase(std::unique(cuts.begin(), cuts.end()), cuts.end());
  auto find = [](const std::vector<Digit>& v, int64_t lo, int64_t hi, int64_t* stride) {
    for (const Digit& d : v) {
      if (d.pos <= lo && hi <= d.pos * d.mod) {
        if (lo % d.pos) return false;
        *stride = d.stride * (lo / d.pos);
        return true;
      }
    }
    return false;
  };
  std::vector<PairDigit> r;
  for (size_t i = 0; i + 1 < cuts.size(); ++i) {
    const int64_t lo = cuts[i], hi = cuts[i + 1];
    if (hi % lo) return false;
    PairDigit pd{lo, hi / lo, 0, 0};
    const bool in_a = find(a, lo, hi, &pd.sa);
    const bool in_b = find(b, lo, hi, &pd.sb);
    if (in_a != in_b) return false;
    if (!in_a) continue;  // a gap left by size-1 logical dims on both sides
    r.push_back(pd);
  }
  out->swap(r);
  return true;
}

void merge_pairs(std::vector<PairDigit>* v) {
  std::sort(v->begin(), v->end(), [](const PairDigit& x, const PairDigit& y) { return x.sa < y.sa; });
  std::vector<PairDigit> r;
  for (const PairDigit& pd : *v) {
    if (!r.empty()) {
      PairDigit& q = r.back();
      if (q.sa * q.radix == pd.sa && q.sb * q.radix == pd.sb) {
        q.radix *= pd.radix;
        continue;
      }
    }
    r.push_back(pd);
  }
  v->swap(r);
}

}  // namespace lego
