// Passes T, B and C of a round, as a fragment that is included INSIDE the kernel that owns the round's
// shared state: from the angular lists and the per-element counts (ws.ang.cnt_a) of the round's central
// atoms to the angular blocks of their feature rows.  A central atom with all counts zero contributes
// nothing (its blocks keep the zeros written before).  Expects in scope: T, `ws` (a __shared__ object
// with a MolAngularShared member `ang`), `lane`, and the constant kRoundCapA (the CAPA of ws.ang).
// It is a fragment and not a function because the function form, although inlined, compiled to a
// kernel that was 6 % slower (measured: 25.6 -> 27.3 us on a 1024-molecule batch).
{
    // ---- T: one table for the groups (central atom, element pair) of the round.  Lane = (central
    // atom, bucket) covers the first eight buckets in one pass; N-O and O-O pairs (buckets 8, 9)
    // are rare and get a second, short pass only when they occur. ----
    int total = 0;
    for (int pass = 0; pass < 2; pass++) {
        const int g = pass == 0 ? lane >> 3 : (lane >> 1) & 3;
        const int bk = pass == 0 ? lane & 7 : 8 + (lane & 1);
        const bool act = pass == 0 || lane < 8;
        const int ta = (kBucketTa >> (2 * bk)) & 3, tb = (kBucketTb >> (2 * bk)) & 3;
        const int4 ca = *reinterpret_cast<const int4*>(&ws.ang.cnt_a[g * kTypes]);
        const int cav[kTypes] = {ca.x, ca.y, ca.z, ca.w};
        const int stv[kTypes] = {0, ca.x, ca.x + ca.y, ca.x + ca.y + ca.z};
        const int na = pick4(cav, ta), nb = pick4(cav, tb);
        const int cnt = act ? (ta == tb ? na * (na - 1) / 2 : na * nb) : 0;
        if (pass == 1 && !__any_sync(kFull, cnt > 0)) break;
        const int pad = (cnt + 3) & ~3;
        int incl = pad;
#pragma unroll
        for (int o = 1; o < kWarp; o <<= 1) {
            const int y = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += y;
        }
        const int off = total + incl - pad;
        if (cnt > 0) {
            MolGroupInfo e;
            e.off = off;
            e.cnt = cnt;
            e.packed = (g * kRoundCapA + pick4(stv, ta)) | ((g * kRoundCapA + pick4(stv, tb)) << 8) | (nb << 16) |
                       ((ta == tb ? 1 : 0) << 24);
            e.recip = (unsigned)(65536.0f * __frcp_rn((float)nb)) + 1u;   // in [2^16 / nb, 2^16 / nb + 1.01)
            const int gid = g * kMolGroupStride + bk;
            ws.ang.tab[gid] = e;
            for (int q = off >> 2; q < (off + pad) >> 2; q++) ws.ang.quad_gid[q] = (unsigned char)gid;
        }
        total += __shfl_sync(kFull, incl, kWarp - 1);
    }
    // ids behind the last group, through the end of its chunk and the look-ahead of pass C
    for (int q = (total >> 2) + lane; q < (((total + kMolChunk - 1) & ~(kMolChunk - 1)) >> 2) + 1; q += kWarp)
        ws.ang.quad_gid[q] = (unsigned char)kMolNoGroup;
    __syncwarp();

    // ---- B + C over the slots of the round ----
    const T* a_row = &ws.ang.A[lane >> 2][0];
    const T* b_row = &ws.ang.BF[lane & 3][0];
    Pair<T> acc0{(T)0, (T)0}, acc1{(T)0, (T)0};
    for (int c0 = 0; c0 < total; c0 += kMolChunk) {
        // B: lane = slot, kMolSlotsPerLane slots per lane (independent of one another)
#pragma unroll
        for (int u = 0; u < kMolSlotsPerLane; u++) {
            int a, b;
            const bool valid = decode_slot(ws.ang.tab, ws.ang.quad_gid, c0 + u * kWarp + lane, &a, &b);
            const Vec4<T> ua = ws.ang.ang_u[a], ub = ws.ang.ang_u[b];
            const T cosv = ua.x * ub.x + ua.y * ub.y + ua.z * ub.z;
            const T rbar = (T)0.5 * (ua.w + ub.w);
            const T fcprod = valid ? ws.ang.ang_fc[a] * ws.ang.ang_fc[b] : (T)0;
            T A[kNumThetas], BF[kNumARs];
            angular_factors_dev<T>(cosv, rbar, fcprod, A, BF);
#pragma unroll
            for (int t = 0; t < kNumThetas; t++) ws.ang.A[t][u * kWarp + lane] = A[t];
#pragma unroll
            for (int q = 0; q < kNumARs; q++) ws.ang.BF[q][u * kWarp + lane] = BF[q];
        }
        // quads of this chunk that end a group (the first lanes look at one quad each)
        const unsigned char* ids = &ws.ang.quad_gid[c0 >> 2];
        constexpr int kQuads = kMolChunk / 4;
        const unsigned my_id = ids[lane & (kQuads - 1)];
        const unsigned ends =
            __ballot_sync(kFull, lane < kQuads && my_id != kMolNoGroup && my_id != ids[(lane & (kQuads - 1)) + 1]);
        __syncwarp();
        // C: lane = (theta, shift).  Slots behind the last group hold BF = 0.
#pragma unroll
        for (int q = 0; q < kQuads; q++) {
            T av[4], bv[4];
            load4(a_row + 4 * q, av);
            load4(b_row + 4 * q, bv);
            acc0 = pfma(Pair<T>{av[0], av[1]}, Pair<T>{bv[0], bv[1]}, acc0);
            acc1 = pfma(Pair<T>{av[2], av[3]}, Pair<T>{bv[2], bv[3]}, acc1);
            if ((ends >> q) & 1u) {
                const unsigned id = ids[q];
                T* row = ws.ang.row[id >> 4];
                row[kRadial + (id & 15u) * kTS + lane] = (acc0.x + acc0.y) + (acc1.x + acc1.y);
                acc0 = Pair<T>{(T)0, (T)0};
                acc1 = Pair<T>{(T)0, (T)0};
            }
        }
        __syncwarp();
    }
}
