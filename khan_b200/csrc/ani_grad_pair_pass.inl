// The pair pass of the gradient kernels, as a fragment that is included inside a kernel (the function
// form of such code compiled measurably worse): the neighbour pairs of every central atom in the warp's
// neighbour list, in circulant order.  The k neighbours of a central atom occupy k consecutive list
// entries = lanes; lane a handles the pair (a, a + d mod k) for d = 1 .. k / 2, keeps the force on a in
// registers and hands the force on b to its owner with one shuffle; spare lanes run further offsets d
// at the same time (`mult` copies of the list side by side).
// Expects in scope: T, `ws` with nb[] (MolGradNeighbor<T>: info = element | ... | first entry of the
// central atom's run << 7 | length of the run << 12 | upstream row buffer << 18 | ...) and g[][] (the
// upstream rows), `lane`, `used` (entries in the list), `max_half` (largest k / 2 in the list, > 0).
// Leaves: `ea` (the entry of this lane, lanes >= used hold a copy of another entry) and fax, fay, faz =
// the force on the neighbour of entry `lane` from all angular terms of its central atom (lanes < used).
    // offsets d that run at once on spare lanes
    const int mult = used * 4 <= kWarp ? 4 : (used * 3 <= kWarp ? 3 : (used * 2 <= kWarp ? 2 : 1));
    const int copy = (lane >= used ? 1 : 0) + (lane >= 2 * used ? 1 : 0) + (lane >= 3 * used ? 1 : 0);
    const bool owner = copy < mult;
    const int l1 = owner ? lane - copy * used : 0;
    const MolGradNeighbor<T> ea = ws.nb[l1];
    const int ta = ea.info & 3, lb = (ea.info >> 7) & 31, na = (ea.info >> 12) & 63;
    const T* gblocks = ws.g[(ea.info >> 18) & 3] + kRadial;
    const int a = l1 - lb, hf = na >> 1;
    const bool even = (na & 1) == 0;
    T fax = (T)0, fay = (T)0, faz = (T)0;   // force on neighbour a, this copy's share
    const int iters = (max_half + mult - 1) / mult;
    for (int it = 0; it < iters; it++) {
        const int d = 1 + copy + it * mult;
        const bool in_range = owner && d <= hf;
        const bool valid = in_range && !(even && d == hf && a >= hf);
        int b = a + d;
        if (b >= na) b -= na;
        T gbx = (T)0, gby = (T)0, gbz = (T)0;
        if (valid) {
            const MolGradNeighbor<T> eb = ws.nb[lb + b];
            T c = ea.u.x * eb.u.x + ea.u.y * eb.u.y + ea.u.z * eb.u.z;
            c = Num<T>::max_((T)-1, Num<T>::min_((T)1, c));
            const T s2 = sin2_from_cross<T>(ea.u.x, ea.u.y, ea.u.z, eb.u.x, eb.u.y, eb.u.z);
            T gl[kTS];
            const T* gsrc = gblocks + bucket_of(ta, eb.info & 3) * kGradBucketStride;
#pragma unroll
            for (int q = 0; q < kTS; q += 4) load4(gsrc + q, gl + q);
            T dc, dra, drb;
            angular_vjp_dev<T>(c, s2, ea.u.w, eb.u.w, ea.fc, ea.dfc, eb.fc, eb.dfc, gl, &dc, &dra, &drb);
            const T aa = -dc * ea.inv_r, ba = c * dc * ea.inv_r - dra;
            const T ab = -dc * eb.inv_r, bb = c * dc * eb.inv_r - drb;
            fax += aa * eb.u.x + ba * ea.u.x;
            fay += aa * eb.u.y + ba * ea.u.y;
            faz += aa * eb.u.z + ba * ea.u.z;
            gbx = ab * ea.u.x + bb * eb.u.x;
            gby = ab * ea.u.y + bb * eb.u.y;
            gbz = ab * ea.u.z + bb * eb.u.z;
        }
        // the force on b goes to the lane that owns b: lane a takes it from the lane
        // of (a - d) mod k in its own copy
        int sa = a - d;
        if (sa < 0) sa += na;
        const int from = in_range ? copy * used + lb + sa : lane;
        fax += __shfl_sync(kFull, gbx, from);
        fay += __shfl_sync(kFull, gby, from);
        faz += __shfl_sync(kFull, gbz, from);
    }
    for (int k2 = 1; k2 < mult; k2++) {   // sum the copies
        const int s = lane + k2 * used;
        const int from = s < kWarp ? s : lane;
        const T ox = __shfl_sync(kFull, fax, from), oy = __shfl_sync(kFull, fay, from),
                oz = __shfl_sync(kFull, faz, from);
        if (lane < used) { fax += ox; fay += oy; faz += oz; }
    }
