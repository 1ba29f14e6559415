// Launch glue of the row forward and backward: argument checks, the decomposition of a call into
// blocks, kernel selection. Included once per translation unit; each unit compiles the row kernels
// for one mask format (NRL_MASK_BITS 0: a byte per token, 1: a bit per token) in its own namespace
// and gives the two entry functions its own names through NRL_ROW_FWD_ENTRY / NRL_ROW_BWD_ENTRY.

// ---- decomposition of the forward -------------------------------------------------------------

// Blocks per row: 1 once there are at least two waves of rows; otherwise enough to reach that,
// keeping at least 16 tiles (4096 elements) per block. A function of (rows, V) only.
static uint32_t fwd_nsplit(uint64_t rows, uint32_t V) {
    const uint64_t want = 2 * 148;
    if (rows >= want) return 1;
    uint32_t tiles = (V + kTile - 1) / kTile;
    uint32_t max_split = tiles / 16;
    if (max_split < 1) max_split = 1;
    if (max_split > 16) max_split = 16;
    uint64_t need = (want + rows - 1) / rows;
    return (uint32_t)(need < max_split ? need : max_split);
}

template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
static int launch_fwd(const FwdParams& p, cudaStream_t st) {
    if (p.nsplit == 1) {
        if constexpr (VEC && !GENERAL) {
            // many rows on a fast path: a block takes a group of rows and overlaps each row's tail
            // with the next rows' streaming
            FwdParams q = p;  // a row in kGroupSplit ranges of kWarps parts each
            q.nsplit = kGroupSplit;
            q.tiles_per_block = (p.tiles_per_block + q.nsplit - 1) / q.nsplit;
            const uint32_t part_vectors = (q.tiles_per_block + q.parts_per_block - 1) / q.parts_per_block * (kTile / kVec);
            if (!(p.flags & (NRL_FWD_GREEDY | NRL_FWD_ROW_PER_BLOCK)) && p.rows >= 2ull * 148 * group_rows<ALLOW>() && part_vectors < 0xffffu && q.tiles_per_block >= 16) {
                row_fwd_grouped<DT, REF, ALLOW><<<(unsigned)((p.rows + group_rows<ALLOW>() - 1) / group_rows<ALLOW>()), kThreads, 0, st>>>(q);
                return after_launch();
            }
        }
        row_fwd_fused<DT, REF, ALLOW, GENERAL, VEC><<<(unsigned)p.rows, kThreads, 0, st>>>(p);
        return after_launch();
    }
    row_fwd_parts<DT, REF, ALLOW, GENERAL, VEC><<<(unsigned)(p.rows * p.nsplit), kThreads, 0, st>>>(p);
    int rc = after_launch();
    if (rc) return rc;
    row_fwd_finish<DT, REF, ALLOW, GENERAL, VEC><<<(unsigned)p.rows, kThreads, 0, st>>>(p);
    return after_launch();
}

// GENERAL = additive mask, temperature ≠ 1 or the scalar-load path; VEC = 16-byte loads.
#define NRL_DISPATCH(FN, dt, ref, allow, general, vec, ...)                                                        \
    do {                                                                                                           \
        if (vec && !general) {                                                                                     \
            if (dt == NRL_BF16) { if (ref) { if (allow) return FN<NRL_BF16, true, true, false, true>(__VA_ARGS__); else return FN<NRL_BF16, true, false, false, true>(__VA_ARGS__); } \
                                  else     { if (allow) return FN<NRL_BF16, false, true, false, true>(__VA_ARGS__); else return FN<NRL_BF16, false, false, false, true>(__VA_ARGS__); } } \
            else                { if (ref) { if (allow) return FN<NRL_F32, true, true, false, true>(__VA_ARGS__); else return FN<NRL_F32, true, false, false, true>(__VA_ARGS__); } \
                                  else     { if (allow) return FN<NRL_F32, false, true, false, true>(__VA_ARGS__); else return FN<NRL_F32, false, false, false, true>(__VA_ARGS__); } } \
        } else if (vec) {                                                                                          \
            if (dt == NRL_BF16) { if (ref) { if (allow) return FN<NRL_BF16, true, true, true, true>(__VA_ARGS__); else return FN<NRL_BF16, true, false, true, true>(__VA_ARGS__); } \
                                  else     { if (allow) return FN<NRL_BF16, false, true, true, true>(__VA_ARGS__); else return FN<NRL_BF16, false, false, true, true>(__VA_ARGS__); } } \
            else                { if (ref) { if (allow) return FN<NRL_F32, true, true, true, true>(__VA_ARGS__); else return FN<NRL_F32, true, false, true, true>(__VA_ARGS__); } \
                                  else     { if (allow) return FN<NRL_F32, false, true, true, true>(__VA_ARGS__); else return FN<NRL_F32, false, false, true, true>(__VA_ARGS__); } } \
        } else {                                                                                                   \
            if (dt == NRL_BF16) { if (ref) { if (allow) return FN<NRL_BF16, true, true, true, false>(__VA_ARGS__); else return FN<NRL_BF16, true, false, true, false>(__VA_ARGS__); } \
                                  else     { if (allow) return FN<NRL_BF16, false, true, true, false>(__VA_ARGS__); else return FN<NRL_BF16, false, false, true, false>(__VA_ARGS__); } } \
            else                { if (ref) { if (allow) return FN<NRL_F32, true, true, true, false>(__VA_ARGS__); else return FN<NRL_F32, true, false, true, false>(__VA_ARGS__); } \
                                  else     { if (allow) return FN<NRL_F32, false, true, true, false>(__VA_ARGS__); else return FN<NRL_F32, false, false, true, false>(__VA_ARGS__); } } \
        }                                                                                                          \
    } while (0)

static bool aligned16(uint64_t p) { return (p & 15u) == 0; }

// Can every stream of this call use 16-byte (8-byte for the byte mask) vector loads?
static bool can_vectorise(uint32_t V, uint64_t logits, uint64_t ref, uint64_t allow, uint64_t allow_stride, uint64_t add, uint64_t add_stride) {
    if (V % kVec != 0) return false;
    if (!aligned16(logits) || (ref && !aligned16(ref))) return false;
#if !NRL_MASK_BITS
    if (allow && ((allow & 7u) != 0 || allow_stride % kVec != 0)) return false;
#endif
    if (add && (!aligned16(add) || add_stride % 4 != 0)) return false;
    return true;
}

static int fill_fwd_params(FwdParams& p, uint32_t dtype, uint32_t V, uint64_t rows, float tau, uint64_t logits, uint64_t ref, uint64_t allow, uint64_t allow_stride,
                           uint64_t add, uint64_t add_stride) {
    if (rows == 0 || V == 0 || !logits) return NRL_E_BAD_ARG;
    if (dtype != NRL_F32 && dtype != NRL_BF16) return NRL_E_UNSUPPORTED;
    if (!(tau > 0.f) || !isfinite(tau)) return NRL_E_BAD_ARG;
#if NRL_MASK_BITS
    // a bit per token: `allow_stride` arrives in 32-bit words between rows (0: one row for all)
    if (!allow || (allow & 3u) || (allow_stride != 0 && allow_stride < (V + 31u) / 32u)) return NRL_E_BAD_ARG;
    allow_stride *= 4;  // the kernels step in bytes
#else
    if (allow && allow_stride != 0 && allow_stride != V) return NRL_E_BAD_ARG;
#endif
    if (add && add_stride != 0 && add_stride != V) return NRL_E_BAD_ARG;
    if ((logits & (dtype == NRL_F32 ? 3u : 1u)) || (ref & (dtype == NRL_F32 ? 3u : 1u)) || (add & 3u)) return NRL_E_BAD_ARG;
    memset(&p, 0, sizeof p);
    p.logits = (const void*)logits;
    p.ref = (const void*)ref;
    p.allow = (const uint8_t*)allow;
    p.add = (const float*)add;
    p.rows = rows;
    p.allow_stride = allow_stride;
    p.add_stride = add_stride;
    p.V = V;
    p.tau = tau;
    p.nsplit = 1;
    p.tiles_per_block = (V + kTile - 1) / kTile;
    p.parts_per_block = kWarps;
    return NRL_OK;
}

static int dispatch_fwd(const FwdParams& p, uint32_t dt, bool ref, bool allow, bool general, bool vec, cudaStream_t st) {
    NRL_DISPATCH(launch_fwd, dt, ref, allow, general, vec, p, st);
    return NRL_E_UNSUPPORTED;
}

int NRL_ROW_FWD_ENTRY(const nrl_row_fwd_args* a, nrl_stream stream) {
    if (!a || a->struct_size != sizeof(nrl_row_fwd_args)) return NRL_E_BAD_ARG;
    FwdParams p;
    int rc = fill_fwd_params(p, a->dtype, a->V, a->rows, a->temperature, a->logits, a->ref_logits, a->allow_mask, a->allow_row_stride, a->add_mask, a->add_row_stride);
    if (rc) return rc;
    uint32_t mode = a->flags & (NRL_FWD_SAMPLE | NRL_FWD_GREEDY | NRL_FWD_TOKENS_IN);
    if (mode & (mode - 1)) return NRL_E_BAD_ARG;  // more than one mode
    if (a->flags & ~(uint32_t)(NRL_FWD_SAMPLE | NRL_FWD_GREEDY | NRL_FWD_TOKENS_IN | NRL_FWD_ROW_PER_BLOCK | (NRL_MASK_BITS ? NRL_FWD_MASK_BITS : 0u))) return NRL_E_BAD_ARG;
    if ((mode & NRL_FWD_SAMPLE) && !a->uniforms) return NRL_E_BAD_ARG;
    if (mode && !a->tokens) return NRL_E_BAD_ARG;
    if (!mode && (a->logp || a->ref_logp)) return NRL_E_BAD_ARG;  // log-prob of which token?
    if ((a->kl || a->ref_logp) && !a->ref_logits) return NRL_E_BAD_ARG;
    if (a->rowstats & 15u) return NRL_E_BAD_ARG;
    if (a->rows * (uint64_t)16 > 0x7fffffffull) return NRL_E_UNSUPPORTED;  // grid size; callers slice along S
    p.uniforms = (const float*)a->uniforms;
    p.tokens = (int32_t*)a->tokens;
    p.logp = (float*)a->logp;
    p.ref_logp = (float*)a->ref_logp;
    p.kl = (float*)a->kl;
    p.entropy = (float*)a->entropy;
    p.rowstats = (float*)a->rowstats;
    p.status = (uint8_t*)a->status;
    p.flags = a->flags;
    p.nsplit = fwd_nsplit(a->rows, a->V);
    if (p.nsplit > 1) {
        uint64_t need = nrl_row_fwd_workspace_bytes(a->rows, a->V);
        if (!a->workspace || a->workspace_bytes < need || (a->workspace & 15u)) return NRL_E_WORKSPACE;
        p.parts = (float*)a->workspace;
        uint32_t tiles = (a->V + kTile - 1) / kTile;
        p.tiles_per_block = (tiles + p.nsplit - 1) / p.nsplit;
    }
    bool vec = can_vectorise(a->V, a->logits, a->ref_logits, a->allow_mask, a->allow_row_stride, a->add_mask, a->add_row_stride);
    bool general = !vec || a->add_mask != 0 || a->temperature != 1.0f;
    return dispatch_fwd(p, a->dtype, a->ref_logits != 0, a->allow_mask != 0, general, vec, (cudaStream_t)stream);
}

// ---- backward ------------------------------------------------------------------------------------

template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
static int launch_bwd(const BwdParams& p, cudaStream_t st) {
    const unsigned grid = (unsigned)(p.in.rows * p.chunks_per_row);
    const bool extra = p.accumulate || p.g_uni || p.d_ref || !p.d_logits;
    // f32 logits, and bf16 logits alone (the cross-entropy backward): stores and loads that fill whole
    // sectors measured faster. With a mask or a reference stream the 8-element mapping, with its
    // fewer and wider loads, measured as fast or faster, so those stay on it.
    if constexpr (VEC && !GENERAL && !ALLOW && (DT == NRL_F32 || !REF)) {
        if (!extra && aligned16((uint64_t)(uintptr_t)p.d_logits)) {
            row_bwd_split_kernel<DT, REF, ALLOW><<<grid, kBwdThreads, 0, st>>>(p);
            return after_launch();
        }
    }
    // byte- or bit-masked rows on the vectorised path: excluded vectors are zero-filled from the mask alone and the live
    // ones are compacted (measured on the benchmark's grammar masks and on dense random masks)
    if constexpr (VEC && !GENERAL && ALLOW) {
        if (!extra && aligned16((uint64_t)(uintptr_t)p.d_logits)) {
            row_bwd_compact_kernel<DT, REF><<<grid, kBwdThreads, 0, st>>>(p);
            return after_launch();
        }
    }
    if (extra) row_bwd_kernel<DT, REF, ALLOW, GENERAL, VEC, true><<<grid, kBwdThreads, 0, st>>>(p);
    else row_bwd_kernel<DT, REF, ALLOW, GENERAL, VEC, false><<<grid, kBwdThreads, 0, st>>>(p);
    return after_launch();
}

static int dispatch_bwd(const BwdParams& p, uint32_t dt, bool ref, bool allow, bool general, bool vec, cudaStream_t st) {
    NRL_DISPATCH(launch_bwd, dt, ref, allow, general, vec, p, st);
    return NRL_E_UNSUPPORTED;
}

int NRL_ROW_BWD_ENTRY(const nrl_row_bwd_args* a, nrl_stream stream) {
    if (!a || a->struct_size != sizeof(nrl_row_bwd_args)) return NRL_E_BAD_ARG;
    BwdParams p;
    memset(&p, 0, sizeof p);
    int rc = fill_fwd_params(p.in, a->dtype, a->V, a->rows, a->temperature, a->logits, a->ref_logits, a->allow_mask, a->allow_row_stride, a->add_mask, a->add_row_stride);
    if (rc) return rc;
    if ((!a->d_logits && !a->d_ref_logits) || !a->rowstats || (a->rowstats & 15u) || (a->d_logits & 3u) || (a->d_ref_logits & 3u)) return NRL_E_BAD_ARG;
    if (a->d_ref_logits && (!a->ref_logits || !a->g_kl)) return NRL_E_BAD_ARG;
    if (a->g_uniform && (a->allow_mask || a->add_mask || a->temperature != 1.0f)) return NRL_E_UNSUPPORTED;
    if (a->g_logp && !a->tokens) return NRL_E_BAD_ARG;
    if (a->g_kl && (!a->ref_logits || !a->kl)) return NRL_E_BAD_ARG;
    if (a->g_ent && !a->entropy) return NRL_E_BAD_ARG;
    p.tokens = (const int32_t*)a->tokens;
    p.rowstats = (const float*)a->rowstats;
    p.kl = (const float*)a->kl;
    p.entropy = (const float*)a->entropy;
    p.g_logp = (const float*)a->g_logp;
    p.g_kl = (const float*)a->g_kl;
    p.g_ent = (const float*)a->g_ent;
    p.g_uni = (const float*)a->g_uniform;
    p.d_logits = (float*)a->d_logits;
    p.d_ref = (float*)a->d_ref_logits;
    p.accumulate = a->accumulate ? 1u : 0u;
    // blocks per row: about 16K elements each, so short rows are one block and long rows spread out
    uint32_t chunks = (a->V + 16383) / 16384;
    if (chunks < 1) chunks = 1;
    p.chunks_per_row = chunks;
    if (a->rows * (uint64_t)chunks > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    bool vec = can_vectorise(a->V, a->logits, a->ref_logits, a->allow_mask, a->allow_row_stride, a->add_mask, a->add_row_stride);
    bool general = !vec || a->add_mask != 0 || a->temperature != 1.0f;
    // without an upstream KL gradient the reference stream is not read at all
    bool ref = a->ref_logits != 0 && a->g_kl != 0;
    return dispatch_bwd(p, a->dtype, ref, a->allow_mask != 0, general, vec, (cudaStream_t)stream);
}

