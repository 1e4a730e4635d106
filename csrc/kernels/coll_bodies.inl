// Bodies of the push-style collectives.  This file is included twice: by collectives.cu
// inside namespace amem::dev with AMEM_FN = __device__ __forceinline__ (CUDA kernels), and by
// host_exec.cc inside namespace amem::hostx with AMEM_FN = inline (the mock backend runs the
// very same protocol on the calling thread, one "block" of one "thread").  The enclosing
// namespace supplies Proto, proto_begin/proto_end, block_barrier, block_sync, block_range,
// copy_span and reduce_span.
//
// Conventions: `es` = bytes per input element, every staging offset is a multiple of 256
// bytes, block ranges start on 16-byte boundaries, `p.opseq` picks the staging half and the
// chunk index picks the quarter inside it.
// Reference parity: stands in for the NCCL collectives the reference guards and exercises
// (nccl_patch/nccl_2.27.5-1.diff:113-230; run.sh:22: all_reduce, all_gather, alltoall, broadcast).

// Peer visited at step k (1..n-1) by `block`; different blocks start at different peers so
// that the stores of one rank fan out over all NVLink destinations at once.
AMEM_FN int peer_at(int rank, int n, int k, int block) { return (rank + 1 + (k - 1 + block) % (n - 1)) % n; }

// All-gather, all-to-all and reduce-scatter share one skeleton: every chunk is PUSHED into the
// peers' staging (NVLink-bound) and then DRAINED from my own staging into the user's buffer
// (HBM-bound).  A message of one chunk does push, one cross-rank barrier, drain.  A longer
// message runs the two jobs on two groups of warps that never meet: they are coupled only by
// per-block credits (CtrlBlock::ready / freed).  The pusher announces chunk N to each peer and
// moves on; it only waits when it is about to overwrite quarter N % 2, for the peers' "drained
// chunk N-2".  The drainer waits for every peer's chunk N, drains it and hands the quarter
// back.  So the link never idles on a barrier, and the drain hides behind the next push.  The
// operation ends when all peers have drained all of my chunks: staging is then free everywhere,
// whatever protocol the next operation uses.
// `with_self`: the two groups of THIS rank also depend on each other (NVLS all-reduce), so the
// credit is sent to, and awaited from, my own control block as well.
AMEM_FN void credit_wait(Proto& p, bool want_ready, uint32_t want, Lane ln, bool with_self = false) {
  const CollArgs& a = *p.a;
  for (int q = ln.tid; q < a.nranks; q += ln.nt) {
    if (q == a.rank && !with_self) continue;
    const uint32_t* f = want_ready ? &p.me->ready[p.block][q] : &p.me->freed[p.block][q];
    if (*(volatile int*)p.abort_flag == 0 && !wait_flag_ge(f, want, a.timeout_ns)) {
      report_error(a.status, kDevBarrierTimeout, a.rank, q, p.block, want);
      *(volatile int*)p.abort_flag = 1;
    }
  }
  lane_sync(ln);
}
AMEM_FN void credit_signal(Proto& p, bool is_ready, uint32_t value, Lane ln, bool with_self = false) {
  const CollArgs& a = *p.a;
  lane_sync(ln);  // everything the group stored (or finished reading) comes before the signal
  for (int q = ln.tid; q < a.nranks; q += ln.nt) {
    if (q == a.rank && !with_self) continue;
    fence_system();
    st_release_sys(is_ready ? &a.ctrl[q]->ready[p.block][a.rank] : &a.ctrl[q]->freed[p.block][a.rank], value);
  }
}

template <typename PushF, typename DrainF>
AMEM_FN void run_chunks(const CollArgs& a, Proto& p, uint32_t nch, int push_sixteenths, PushF push, DrainF drain) {
  if (nch == 0) return;
  if (nch == 1) {
    push(0u, full_lane());
    block_barrier(p);
    drain(0u, full_lane());
    return;
  }
  Lane lp, ld;
  bool do_push, do_drain;
  split_lanes(true, push_sixteenths, &lp, &ld, &do_push, &do_drain);
  const uint32_t base = ld_volatile(&p.me->cseq[p.block]);
  auto push_step = [&](uint32_t t) {
    if (t >= 2) credit_wait(p, false, base + t - 1u, lp);  // peers drained chunk t-2: its quarter is free
    push(t, lp);
    credit_signal(p, true, base + t + 1u, lp);
  };
  auto drain_step = [&](uint32_t t) {
    credit_wait(p, true, base + t + 1u, ld);
    drain(t, ld);
    credit_signal(p, false, base + t + 1u, ld);
  };
  if (lanes_split(lp)) {
    if (do_push) {
      for (uint32_t t = 0; t < nch; ++t) push_step(t);
      credit_wait(p, false, base + nch, lp);
    } else {
      for (uint32_t t = 0; t < nch; ++t) drain_step(t);
    }
  } else {  // one thread plays both groups (host executor)
    for (uint32_t t = 0; t < nch; ++t) {
      push_step(t);
      drain_step(t);
    }
    credit_wait(p, false, base + nch, lp);
  }
  block_sync();
  if (thread_index() == 0) p.me->cseq[p.block] = base + nch;
}

template <typename TI, typename TO, int OP>
AMEM_BODY void body_allgather(const CollArgs& a, Proto& p, size_t chunk_elems) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(TI);
  const size_t B = a.count * es;  // bytes contributed by each rank
  const size_t Q = quarter_bytes(a.stage_bytes, a.p2p_slot_bytes);
  const size_t slot = slot_bytes_of(Q, n);
  size_t cb = chunk_elems * es;
  if (cb > slot) cb = slot;
  const char* send = (const char*)a.send;
  char* recv = (char*)a.recv;
  const uint32_t nch = (uint32_t)((B + cb - 1) / cb);
  const size_t fb = nch == 1 ? B : cb;   // what the blocks split: the whole message, or a full chunk (block_range_clip)
  run_chunks(a, p, nch, 8,
    [&](uint32_t t, Lane ln) {
      size_t off = (size_t)t * cb;
      size_t len = B - off < cb ? B - off : cb;
      size_t qoff = quarter_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq, t);
      size_t lo, hi;
      block_range_clip(fb, len, p.block, p.nblocks, &lo, &hi);
      char* mc = (a.algo == kAlgoNvls && a.mc_stage) ? a.mc_stage + qoff + (size_t)r * slot + lo : nullptr;
      if (mc_copy_ok(mc, send + off + lo, hi - lo)) {
        // NVLS all-gather: one multicast store lands my piece in every rank's staging slot
        copy_span_mc(mc, send + off + lo, hi - lo, ln);
      } else {
        for (int k = 1; k < n; ++k) {
          int q = peer_at(r, n, k, p.block);
          copy_span(a.stage[q] + qoff + (size_t)r * slot + lo, send + off + lo, hi - lo, ln);
        }
      }
      if (send != recv + (size_t)r * B) copy_span(recv + (size_t)r * B + off + lo, send + off + lo, hi - lo, ln);
    },
    [&](uint32_t t, Lane ln) {
      size_t off = (size_t)t * cb;
      size_t len = B - off < cb ? B - off : cb;
      size_t qoff = quarter_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq, t);
      size_t lo, hi;
      block_range_clip(fb, len, p.block, p.nblocks, &lo, &hi);
      for (int k = 1; k < n; ++k) {
        int q = peer_at(r, n, k, p.block);
        copy_span(recv + (size_t)q * B + off + lo, a.stage[r] + qoff + (size_t)q * slot + lo, hi - lo, ln);
      }
    });
}

template <typename TI, typename TO, int OP>
AMEM_BODY void body_alltoall(const CollArgs& a, Proto& p, size_t chunk_elems) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(TI);
  const size_t B = a.count * es;  // bytes exchanged with each peer
  const size_t Q = quarter_bytes(a.stage_bytes, a.p2p_slot_bytes);
  const size_t slot = slot_bytes_of(Q, n);
  size_t cb = chunk_elems * es;
  if (cb > slot) cb = slot;
  const char* send = (const char*)a.send;
  char* recv = (char*)a.recv;
  const uint32_t nch = (uint32_t)((B + cb - 1) / cb);
  const size_t fb = nch == 1 ? B : cb;   // what the blocks split: the whole message, or a full chunk (block_range_clip)
  run_chunks(a, p, nch, 8,
    [&](uint32_t t, Lane ln) {
      size_t off = (size_t)t * cb;
      size_t len = B - off < cb ? B - off : cb;
      size_t qoff = quarter_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq, t);
      size_t lo, hi;
      block_range_clip(fb, len, p.block, p.nblocks, &lo, &hi);
      for (int k = 1; k < n; ++k) {
        int q = peer_at(r, n, k, p.block);
        copy_span(a.stage[q] + qoff + (size_t)r * slot + lo, send + (size_t)q * B + off + lo, hi - lo, ln);
      }
      if (send != recv) copy_span(recv + (size_t)r * B + off + lo, send + (size_t)r * B + off + lo, hi - lo, ln);
    },
    [&](uint32_t t, Lane ln) {
      size_t off = (size_t)t * cb;
      size_t len = B - off < cb ? B - off : cb;
      size_t qoff = quarter_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq, t);
      size_t lo, hi;
      block_range_clip(fb, len, p.block, p.nblocks, &lo, &hi);
      for (int k = 1; k < n; ++k) {
        int q = peer_at(r, n, k, p.block);
        copy_span(recv + (size_t)q * B + off + lo, a.stage[r] + qoff + (size_t)q * slot + lo, hi - lo, ln);
      }
    });
}

// Small all-to-all without a barrier: every 4 bytes travel in an 8-byte packet together with the
// operation's flag, straight into the receiver's flag-in-data slot for this source; the receiver
// polls the packets and copies the payload out.  Nothing orders "data" before "signal" because they
// are the same store.  Slots alternate between two parities; a slot is rewritten two operations
// later, and only after the receiver has acknowledged the earlier one (CtrlBlock::ll_ack), an
// acknowledgement that normally arrived long before it is looked at.  The flag is the block's
// operation count, which starts at 1: zeroed memory never looks like a packet.
template <typename TI, typename TO, int OP>
AMEM_BODY void body_alltoall_ll(const CollArgs& a, Proto& p) {
  const int n = a.nranks, r = a.rank;
  const size_t B = a.count * sizeof(TI);          // bytes exchanged with each peer
  const size_t words = (B + 3) / 4;
  const uint32_t L = ld_volatile(&p.me->ll_seq[p.block]) + 1u;
  const int tid = thread_index();
  const Lane ln = full_lane();
  // words [w0, w1) of every peer's block are this block's share
  const size_t per = (words + p.nblocks - 1) / p.nblocks;
  size_t w0 = (size_t)p.block * per, w1 = w0 + per;
  if (w0 > words) w0 = words;
  if (w1 > words) w1 = words;
  const char* send = (const char*)a.send;
  char* recv = (char*)a.recv;
  if (L > 2u) {  // my operation L-2 used the slots I am about to overwrite
    for (int q = tid; q < n; q += ln.nt) {
      if (q == r) continue;
      if (*(volatile int*)p.abort_flag == 0 && !wait_flag_ge(&p.me->ll_ack[p.block][q], L - 2u, a.timeout_ns)) {
        report_error(a.status, kDevBarrierTimeout, a.rank, q, p.block, L);
        *(volatile int*)p.abort_flag = 1;
      }
    }
    block_sync();
  }
  auto word_of = [&](const char* base, size_t w) -> uint32_t {
    if (w * 4 + 4 <= B && (((uintptr_t)base) & 3) == 0) return *(const uint32_t*)(base + w * 4);
    uint32_t v = 0;
    for (size_t b = 0; b < 4 && w * 4 + b < B; ++b) v |= (uint32_t)(unsigned char)base[w * 4 + b] << (8 * b);
    return v;
  };
  for (int k = 1; k < n; ++k) {
    const int q = peer_at(r, n, k, p.block);
    char* dst = a.stage[q] + ll_slot_offset(a.stage_bytes, a.p2p_slot_bytes, r, L);
    const char* src = send + (size_t)q * B;
    for (size_t w = w0 + tid; w < w1; w += ln.nt) ll_store(dst + w * 8, word_of(src, w), L);
  }
  if (send != recv) copy_span(recv + (size_t)r * B + w0 * 4, send + (size_t)r * B + w0 * 4, (w1 * 4 < B ? w1 * 4 : B) - (w0 * 4 < B ? w0 * 4 : B), ln);
  for (int k = 1; k < n; ++k) {
    const int q = peer_at(r, n, k, p.block);
    const char* src = a.stage[r] + ll_slot_offset(a.stage_bytes, a.p2p_slot_bytes, q, L);
    char* dst = recv + (size_t)q * B;
    for (size_t w = w0 + tid; w < w1; w += ln.nt) {
      uint32_t v = 0;
      if (*(volatile int*)p.abort_flag != 0) break;
      if (!ll_wait(src + w * 8, L, &v, a.timeout_ns)) {
        report_error(a.status, kDevBarrierTimeout, a.rank, q, p.block, L);
        *(volatile int*)p.abort_flag = 1;
        break;
      }
      if (w * 4 + 4 <= B && (((uintptr_t)dst) & 3) == 0) {
        *(uint32_t*)(dst + w * 4) = v;
      } else {
        for (size_t b = 0; b < 4 && w * 4 + b < B; ++b) dst[w * 4 + b] = (char)(v >> (8 * b));
      }
    }
  }
  block_sync();  // every thread has taken its packets out of the slots
  for (int q = tid; q < n; q += ln.nt)
    if (q != r) st_release_sys(&a.ctrl[q]->ll_ack[p.block][r], L);
  if (tid == 0) p.me->ll_seq[p.block] = L;
}

// Reduce-scatter with the optional fused scale and output-type cast (gradient averaging and
// fp32 <-> bf16 conversion happen in the same pass that reduces).
template <typename TI, typename TO, int OP>
AMEM_BODY void body_reducescatter(const CollArgs& a, Proto& p, size_t chunk_elems) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(TI);
  const size_t R = a.count;  // elements each rank receives
  const size_t Q = quarter_bytes(a.stage_bytes, a.p2p_slot_bytes);
  const size_t slot = slot_bytes_of(Q, n);
  size_t ce = chunk_elems;
  if (ce * es > slot) ce = slot / es;
  const char* send = (const char*)a.send;
  TO* recv = (TO*)a.recv;
  const uint32_t nch = (uint32_t)((R + ce - 1) / ce);
  const size_t fe = nch == 1 ? R : ce;   // what the blocks split: the whole message, or a full chunk (block_range_clip)
  // the reduce side reads n slots per output: it gets more warps than the push side
  run_chunks(a, p, nch, 6,
    [&](uint32_t t, Lane ln) {
      size_t off = (size_t)t * ce;
      size_t len = R - off < ce ? R - off : ce;
      size_t qoff = quarter_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq, t);
      size_t lo, hi;
      block_range_clip(fe * es, len * es, p.block, p.nblocks, &lo, &hi);
      for (int k = 1; k < n; ++k) {
        int q = peer_at(r, n, k, p.block);
        copy_span(a.stage[q] + qoff + (size_t)r * slot + lo, send + ((size_t)q * R + off) * es + lo, hi - lo, ln);
      }
    },
    [&](uint32_t t, Lane ln) {
      size_t off = (size_t)t * ce;
      size_t len = R - off < ce ? R - off : ce;
      size_t qoff = quarter_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq, t);
      size_t lo, hi;
      block_range_clip(fe * es, len * es, p.block, p.nblocks, &lo, &hi);
      const TI* slots[kMaxRanks];
      for (int s2 = 0; s2 < n; ++s2)
        slots[s2] = (s2 == r) ? (const TI*)(send + ((size_t)r * R + off) * es + lo)
                              : (const TI*)(a.stage[r] + qoff + (size_t)s2 * slot + lo);
      reduce_span<TI, TO, OP>(recv + off + lo / es, slots, n, (hi - lo) / es, a.scale, a.has_scale != 0, ln);
    });
}

template <typename TI, typename TO, int OP>
AMEM_BODY void body_allreduce_oneshot(const CollArgs& a, Proto& p) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(TI);
  const size_t B = a.count * es;
  const size_t Q = quarter_bytes(a.stage_bytes, a.p2p_slot_bytes);
  const size_t slot = slot_bytes_of(Q, n);
  const char* send = (const char*)a.send;
  size_t qoff = quarter_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq, 0);
  size_t lo, hi;
  block_range(B, p.block, p.nblocks, &lo, &hi);
  for (int k = 1; k < n; ++k) {
    int q = peer_at(r, n, k, p.block);
    copy_span(a.stage[q] + qoff + (size_t)r * slot + lo, send + lo, hi - lo, full_lane());
  }
  block_barrier(p);
  const TI* slots[kMaxRanks];
  for (int s = 0; s < n; ++s)
    slots[s] = (s == r) ? (const TI*)(send + lo) : (const TI*)(a.stage[r] + qoff + (size_t)s * slot + lo);
  reduce_span<TI, TO, OP>((TO*)a.recv + lo / es, slots, n, (hi - lo) / es, a.scale, a.has_scale != 0, full_lane());
}

// All-reduce on registered windows, without staging: every rank's input is mapped here, so rank r
// reduces slice r straight out of the peers' memory (loads over NVLink) into its own output and
// then stores the reduced slice into every peer's output.  One barrier before (the inputs are
// complete: each rank's earlier kernels have finished once its block arrives) and one after (the
// outputs are complete).  Safe in place: slice r is read and written by rank r only.
template <typename TI, typename TO, int OP>
AMEM_BODY void body_allreduce_window(const CollArgs& a, Proto& p) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(TI), vi = 16 / es;
  const size_t N = a.count;
  size_t sl = ((N + n - 1) / n + vi - 1) / vi * vi;
  size_t b0 = (size_t)r * sl, b1 = b0 + sl;
  if (b0 > N) b0 = N;
  if (b1 > N) b1 = N;
  size_t lo, hi;
  block_range((b1 - b0) * es, p.block, p.nblocks, &lo, &hi);
  block_barrier(p);
  const TI* slots[kMaxRanks];
  for (int s2 = 0; s2 < n; ++s2) slots[s2] = (const TI*)(a.win_send[s2] + b0 * es + lo);
  TO* mine = (TO*)(a.win_recv[r] + b0 * es + lo);
  reduce_span<TI, TO, OP>(mine, slots, n, (hi - lo) / es, a.scale, a.has_scale != 0, full_lane());
  block_sync();
  for (int k = 1; k < n; ++k) {
    int q = peer_at(r, n, k, p.block);
    copy_span(a.win_recv[q] + b0 * es + lo, (const char*)mine, hi - lo, full_lane());
  }
  block_barrier(p);
}

template <typename TI, typename TO, int OP>
AMEM_BODY void body_allreduce_twoshot_pipelined(const CollArgs& a, Proto& p, size_t ce, uint32_t nch);

// Two-shot: reduce-scatter of the chunk into region X, then all-gather of the reduced slices
// through region Y; both regions live in the half selected by opseq, no quarter alternation
// is needed because each chunk ends with a barrier of its own before Y is read.
template <typename TI, typename TO, int OP>
AMEM_BODY void body_allreduce_twoshot(const CollArgs& a, Proto& p, size_t chunk_elems) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(TI);
  const size_t N = a.count;
  const size_t H = 2 * quarter_bytes(a.stage_bytes, a.p2p_slot_bytes);
  const size_t slot = slot_bytes_of(H / 2, n);
  const size_t hoff = half_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq);
  const size_t xoff = hoff, yoff = hoff + H / 2;
  const size_t vi = 16 / es;
  size_t ce = chunk_elems;
  if (ce > (slot / es) * n) ce = (slot / es) * n;
  ce = ce / (vi * n) * (vi * n);
  if (ce == 0) ce = vi * n;
  const char* send = (const char*)a.send;
  char* recv = (char*)a.recv;
  {
    // several chunks: the credit pipeline (its buffers are half as large, so re-chunk for it)
    const size_t slot2 = slot_bytes_of(quarter_bytes(a.stage_bytes, a.p2p_slot_bytes) / 2, n);
    size_t ce2 = chunk_elems;
    if (ce2 > (slot2 / es) * n) ce2 = (slot2 / es) * n;
    ce2 = ce2 / (vi * n) * (vi * n);
    if (ce2 == 0) ce2 = vi * n;
    const uint32_t nch2 = (uint32_t)((N + ce2 - 1) / ce2);
    if (nch2 > 1) {
      body_allreduce_twoshot_pipelined<TI, TO, OP>(a, p, ce2, nch2);
      return;
    }
  }
  for (size_t off = 0; off < N; off += ce) {
    size_t len = N - off < ce ? N - off : ce;
    // slice length: equal parts rounded up to a whole 16-byte vector
    size_t sl = ((len + n - 1) / n + vi - 1) / vi * vi;
    for (int k = 1; k < n; ++k) {
      int q = peer_at(r, n, k, p.block);
      size_t b0 = (size_t)q * sl, b1 = b0 + sl;
      if (b0 > len) b0 = len;
      if (b1 > len) b1 = len;
      size_t lo, hi;
      block_range((b1 - b0) * es, p.block, p.nblocks, &lo, &hi);
      copy_span(a.stage[q] + xoff + (size_t)r * slot + lo, send + (off + b0) * es + lo, hi - lo, full_lane());
    }
    block_barrier(p);
    {
      size_t b0 = (size_t)r * sl, b1 = b0 + sl;
      if (b0 > len) b0 = len;
      if (b1 > len) b1 = len;
      size_t lo, hi;
      block_range((b1 - b0) * es, p.block, p.nblocks, &lo, &hi);
      const TI* slots[kMaxRanks];
      for (int s = 0; s < n; ++s)
        slots[s] = (s == r) ? (const TI*)(send + (off + b0) * es + lo)
                            : (const TI*)(a.stage[r] + xoff + (size_t)s * slot + lo);
      char* mine = a.stage[r] + yoff + (size_t)r * slot + lo;
      reduce_span<TI, TO, OP>((TO*)mine, slots, n, (hi - lo) / es, a.scale, a.has_scale != 0, full_lane());
      block_sync();
      for (int k = 1; k < n; ++k) {
        int q = peer_at(r, n, k, p.block);
        copy_span(a.stage[q] + yoff + (size_t)r * slot + lo, mine, hi - lo, full_lane());
      }
      copy_span(recv + (off + b0) * es + lo, mine, hi - lo, full_lane());
    }
    block_barrier(p);
    for (int k = 1; k < n; ++k) {
      int q = peer_at(r, n, k, p.block);
      size_t b0 = (size_t)q * sl, b1 = b0 + sl;
      if (b0 > len) b0 = len;
      if (b1 > len) b1 = len;
      size_t lo, hi;
      block_range((b1 - b0) * es, p.block, p.nblocks, &lo, &hi);
      copy_span(recv + (off + b0) * es + lo, a.stage[r] + yoff + (size_t)q * slot + lo, hi - lo, full_lane());
    }
  }
}

// Two-shot all-reduce for messages of several chunks, on credits.  Per chunk: (1) SCATTER my
// copy of every slice to its owner's X region, (2) the owner REDUCEs its slice (its own
// copy straight from the user's buffer, the others from X) and stores the result into every
// rank's Y region and its own output, (3) every rank GATHERs the other slices from Y into its
// output.  One group of warps does (1) and (3), the other does (2); "scattered N" (ready) and
// "reduced N" (freed) credits, also between the two groups of one rank, couple them.  X and Y
// are double buffered: a buffer is rewritten two chunks later, which the credit order makes
// safe (scatter of N waits for everybody's reduce of N-2; the reduce of N waits for everybody's
// scatter of N, which each rank issues after its gather of N-2).
template <typename TI, typename TO, int OP>
AMEM_BODY void body_allreduce_twoshot_pipelined(const CollArgs& a, Proto& p, size_t ce, uint32_t nch) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(TI), vi = 16 / es;
  const size_t N = a.count;
  const size_t Q = quarter_bytes(a.stage_bytes, a.p2p_slot_bytes);
  const size_t hoff = half_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq);
  const size_t slot = slot_bytes_of(Q / 2, n);  // X and Y each hold two buffers of n slots
  const char* send = (const char*)a.send;
  char* recv = (char*)a.recv;
  auto xbase = [&](uint32_t t) { return hoff + (size_t)(t & 1u) * (Q / 2); };
  auto ybase = [&](uint32_t t) { return hoff + Q + (size_t)(t & 1u) * (Q / 2); };
  // Slices and block ranges are those of a FULL chunk in every chunk (a short last chunk just fills
  // fewer of them): block b then touches the same bytes of X and Y each time, which is what lets
  // per-block credits order the reuse of a buffer two chunks later (see block_range_clip).
  const size_t sl_full = ((ce + n - 1) / n + vi - 1) / vi * vi;
  auto slice = [&](uint32_t t, int owner, size_t* off, size_t* b0, size_t* b1) {
    *off = (size_t)t * ce;
    size_t len = N - *off < ce ? N - *off : ce;
    *b0 = (size_t)owner * sl_full;
    *b1 = *b0 + sl_full;
    if (*b0 > len) *b0 = len;
    if (*b1 > len) *b1 = len;
  };
  auto scatter = [&](uint32_t t, Lane ln) {
    for (int k = 1; k < n; ++k) {
      int q = peer_at(r, n, k, p.block);
      size_t off, b0, b1, lo, hi;
      slice(t, q, &off, &b0, &b1);
      block_range_clip(sl_full * es, (b1 - b0) * es, p.block, p.nblocks, &lo, &hi);
      copy_span(a.stage[q] + xbase(t) + (size_t)r * slot + lo, send + (off + b0) * es + lo, hi - lo, ln);
    }
  };
  auto reduce = [&](uint32_t t, Lane ln) {
    size_t off, b0, b1, lo, hi;
    slice(t, r, &off, &b0, &b1);
    block_range_clip(sl_full * es, (b1 - b0) * es, p.block, p.nblocks, &lo, &hi);
    const TI* slots[kMaxRanks];
    for (int s2 = 0; s2 < n; ++s2)
      slots[s2] = (s2 == r) ? (const TI*)(send + (off + b0) * es + lo) : (const TI*)(a.stage[r] + xbase(t) + (size_t)s2 * slot + lo);
    char* mine = a.stage[r] + ybase(t) + (size_t)r * slot + lo;
    reduce_span<TI, TO, OP>((TO*)mine, slots, n, (hi - lo) / es, a.scale, a.has_scale != 0, ln);
    lane_sync(ln);
    for (int k = 1; k < n; ++k) {
      int q = peer_at(r, n, k, p.block);
      copy_span(a.stage[q] + ybase(t) + (size_t)r * slot + lo, mine, hi - lo, ln);
    }
    copy_span(recv + (off + b0) * es + lo, mine, hi - lo, ln);
  };
  auto gather = [&](uint32_t t, Lane ln) {
    for (int k = 1; k < n; ++k) {
      int q = peer_at(r, n, k, p.block);
      size_t off, b0, b1, lo, hi;
      slice(t, q, &off, &b0, &b1);
      block_range_clip(sl_full * es, (b1 - b0) * es, p.block, p.nblocks, &lo, &hi);
      copy_span(recv + (off + b0) * es + lo, a.stage[r] + ybase(t) + (size_t)q * slot + lo, hi - lo, ln);
    }
  };
  Lane lr, lc;
  bool do_red, do_copy;
  split_lanes(true, 8, &lr, &lc, &do_red, &do_copy);
  const uint32_t base = ld_volatile(&p.me->cseq[p.block]);
  auto copy_step = [&](uint32_t t) {   // t runs to nch + 1
    if (t >= 2) {
      credit_wait(p, false, base + (t - 2) + 1u, lc, true);   // every rank reduced chunk t-2
      gather(t - 2, lc);
    }
    if (t < nch) {
      scatter(t, lc);
      credit_signal(p, true, base + t + 1u, lc, true);        // "scattered t"
    }
  };
  auto reduce_step = [&](uint32_t t) {
    credit_wait(p, true, base + t + 1u, lr, true);
    reduce(t, lr);
    credit_signal(p, false, base + t + 1u, lr, true);          // "reduced t"
  };
  if (lanes_split(lr)) {
    if (do_copy) {
      for (uint32_t t = 0; t < nch + 2; ++t) copy_step(t);
    } else {
      for (uint32_t t = 0; t < nch; ++t) reduce_step(t);
    }
  } else {  // one thread plays both groups (host executor)
    for (uint32_t t = 0; t < nch + 2; ++t) {
      copy_step(t);
      if (t < nch) reduce_step(t);
    }
  }
  block_sync();
  if (thread_index() == 0) p.me->cseq[p.block] = base + nch;
}

// Broadcast.  The root's data goes into every rank's staging — through the multicast mapping when
// there is one (ONE multimem.st per 16 bytes, replicated by the switch: the root's link carries the
// message once, not n - 1 times), by one store per peer otherwise — and every other rank drains its
// staging into its buffer.  Chunks run on the same credits as all-gather: the root's next chunk is
// on the wire while the previous one is drained.
template <typename TI, typename TO, int OP>
AMEM_BODY void body_broadcast(const CollArgs& a, Proto& p, size_t chunk_elems) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(TI);
  const size_t B = a.count * es;
  const size_t Q = quarter_bytes(a.stage_bytes, a.p2p_slot_bytes);
  size_t cb = chunk_elems * es;
  if (cb > Q) cb = Q;
  cb &= ~(size_t)255;
  if (cb == 0) cb = 256;
  const char* send = (const char*)a.send;
  char* recv = (char*)a.recv;
  const uint32_t nch = (uint32_t)((B + cb - 1) / cb);
  const size_t fb = nch == 1 ? B : cb;   // what the blocks split: the whole message, or a full chunk (block_range_clip)
  // The root only pushes and the others only drain: give nearly all warps of a block to the job
  // this rank has (the other group just passes the credits on).
  run_chunks(a, p, nch, r == a.root ? 15 : 1,
    [&](uint32_t t, Lane ln) {
      if (r != a.root) return;
      size_t off = (size_t)t * cb;
      size_t len = B - off < cb ? B - off : cb;
      size_t qoff = quarter_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq, t);
      size_t lo, hi;
      block_range_clip(fb, len, p.block, p.nblocks, &lo, &hi);
      char* mc = (n > 2 && a.mc_stage) ? a.mc_stage + qoff + lo : nullptr;
      if (mc_copy_ok(mc, send + off + lo, hi - lo)) {
        copy_span_mc(mc, send + off + lo, hi - lo, ln);
      } else {
        for (int k = 1; k < n; ++k) {
          int q = peer_at(r, n, k, p.block);
          copy_span(a.stage[q] + qoff + lo, send + off + lo, hi - lo, ln);
        }
      }
      if (send != recv) copy_span(recv + off + lo, send + off + lo, hi - lo, ln);
    },
    [&](uint32_t t, Lane ln) {
      if (r == a.root) return;
      size_t off = (size_t)t * cb;
      size_t len = B - off < cb ? B - off : cb;
      size_t qoff = quarter_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq, t);
      size_t lo, hi;
      block_range_clip(fb, len, p.block, p.nblocks, &lo, &hi);
      copy_span(recv + off + lo, a.stage[r] + qoff + lo, hi - lo, ln);
    });
}

template <typename TI, typename TO, int OP>
AMEM_BODY void body_reduce(const CollArgs& a, Proto& p, size_t chunk_elems) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(TI);
  const size_t N = a.count;
  const size_t Q = quarter_bytes(a.stage_bytes, a.p2p_slot_bytes);
  const size_t slot = slot_bytes_of(Q, n);
  size_t ce = chunk_elems;
  if (ce * es > slot) ce = slot / es;
  const char* send = (const char*)a.send;
  const size_t fe = N <= ce ? N : ce;   // what the blocks split: the whole message, or a full chunk (block_range_clip)
  uint32_t c = 0;
  for (size_t off = 0; off < N; off += ce, ++c) {
    size_t len = N - off < ce ? N - off : ce;
    size_t qoff = quarter_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq, c);
    size_t lo, hi;
    block_range_clip(fe * es, len * es, p.block, p.nblocks, &lo, &hi);
    if (r != a.root) copy_span(a.stage[a.root] + qoff + (size_t)r * slot + lo, send + off * es + lo, hi - lo, full_lane());
    block_barrier(p);
    if (r == a.root) {
      const TI* slots[kMaxRanks];
      for (int s = 0; s < n; ++s)
        slots[s] = (s == r) ? (const TI*)(send + off * es + lo) : (const TI*)(a.stage[r] + qoff + (size_t)s * slot + lo);
      reduce_span<TI, TO, OP>((TO*)a.recv + off + lo / es, slots, n, (hi - lo) / es, a.scale, a.has_scale != 0, full_lane());
    }
  }
}

// Grouped point-to-point: a credit protocol per (peer, lane).  The sender may run two
// slots ahead of the receiver; `p2p_ready` (in the receiver's control block) announces a
// filled slot, `p2p_taken` (in the sender's control block) hands it back.
AMEM_FN void body_sendrecv(const CollArgs& a, int entry, int lane, int lanes, int* s_abort) {
  const CollArgs::P2P& e = a.p2p[entry];
  CtrlBlock* me = a.ctrl[a.rank];
  CtrlBlock* pe = a.ctrl[e.peer];
  const size_t slot = a.p2p_slot_bytes;
  const size_t round_bytes = (size_t)lanes * slot;
  if (thread_index() == 0) *s_abort = 0;
  block_sync();
  if (e.is_send) {
    uint32_t seq = ld_volatile(&me->p2p_sent[e.peer][lane]);
    for (size_t base = 0; base < e.bytes; base += round_bytes) {
      size_t off = base + (size_t)lane * slot;
      if (off >= e.bytes) break;
      size_t len = e.bytes - off < slot ? e.bytes - off : slot;
      if (thread_index() == 0 && *(volatile int*)s_abort == 0) {
        if (!wait_flag_ge(&me->p2p_taken[e.peer][lane], seq - 1u, a.timeout_ns)) {
          report_error(a.status, kDevP2PTimeout, a.rank, e.peer, lane, seq);
          *(volatile int*)s_abort = 1;
        }
      }
      block_sync();
      copy_span(a.stage[e.peer] + p2p_slot_offset(a.stage_bytes, slot, a.rank, seq, lane), (const char*)e.src + off, len, full_lane());
      block_sync();
      if (thread_index() == 0) {
        fence_system();
        st_release_sys(&pe->p2p_ready[a.rank][lane], seq + 1u);
      }
      seq += 1u;
    }
    block_sync();
    if (thread_index() == 0) me->p2p_sent[e.peer][lane] = seq;
  } else {
    uint32_t seq = ld_volatile(&me->p2p_rcvd[e.peer][lane]);
    for (size_t base = 0; base < e.bytes; base += round_bytes) {
      size_t off = base + (size_t)lane * slot;
      if (off >= e.bytes) break;
      size_t len = e.bytes - off < slot ? e.bytes - off : slot;
      if (thread_index() == 0 && *(volatile int*)s_abort == 0) {
        if (!wait_flag_ge(&me->p2p_ready[e.peer][lane], seq + 1u, a.timeout_ns)) {
          report_error(a.status, kDevP2PTimeout, a.rank, e.peer, lane, seq);
          *(volatile int*)s_abort = 1;
        }
      }
      block_sync();
      copy_span((char*)e.dst + off, a.stage[a.rank] + p2p_slot_offset(a.stage_bytes, slot, e.peer, seq, lane), len, full_lane());
      block_sync();
      if (thread_index() == 0) {
        fence_system();
        st_release_sys(&pe->p2p_taken[a.rank][lane], seq + 1u);
      }
      seq += 1u;
    }
    block_sync();
    if (thread_index() == 0) me->p2p_rcvd[e.peer][lane] = seq;
  }
}

// REDUCING selects which bodies are compiled into an instantiation: the copy-only
// collectives are instantiated once for bytes, the reducing ones per (type, operator).
template <typename TI, typename TO, int OP, bool REDUCING>
AMEM_FN void run_body(const CollArgs& a, int block, int nblocks, int* s_abort, size_t chunk_elems) {
  Proto p;
  proto_begin(p, a, block, nblocks, s_abort);
  if (a.nranks == 1) {
    // Single rank: every collective degenerates to a (scaled, cast) copy.
    size_t lo, hi;
    block_range(a.count * sizeof(TI), block, nblocks, &lo, &hi);
    const TI* slots[kMaxRanks];
    slots[0] = (const TI*)((const char*)a.send + lo);
    if ((const void*)a.send != (const void*)a.recv || a.has_scale || sizeof(TI) != sizeof(TO))
      reduce_span<TI, TO, OP>((TO*)a.recv + lo / sizeof(TI), slots, 1, (hi - lo) / sizeof(TI), a.scale, a.has_scale != 0, full_lane());
  } else if constexpr (REDUCING) {
    switch (a.kind) {
      case kCollAllReduce:
        if (a.algo == kAlgoOneShot) body_allreduce_oneshot<TI, TO, OP>(a, p);
        else if (a.algo == kAlgoWindow) body_allreduce_window<TI, TO, OP>(a, p);
        else body_allreduce_twoshot<TI, TO, OP>(a, p, chunk_elems);
        break;
      case kCollReduceScatter: body_reducescatter<TI, TO, OP>(a, p, chunk_elems); break;
      case kCollReduce: body_reduce<TI, TO, OP>(a, p, chunk_elems); break;
      default: break;
    }
  } else {
    switch (a.kind) {
      case kCollAllGather: body_allgather<TI, TO, OP>(a, p, chunk_elems); break;
      case kCollBroadcast: body_broadcast<TI, TO, OP>(a, p, chunk_elems); break;
      case kCollAllToAll:
        if (a.algo == kAlgoLL) body_alltoall_ll<TI, TO, OP>(a, p);
        else body_alltoall<TI, TO, OP>(a, p, chunk_elems);
        break;
      default: break;
    }
  }
  proto_end(p);
}
