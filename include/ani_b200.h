/*
 * ani_b200 -- C ABI of the B200 (sm_100a) implementation of khan's ANI-1 featurizer path.
 *
 * Every entry point below takes the place of one piece of the reference's `ani.so`
 * TensorFlow custom-op library (gpu_featurizer/ of proteneer/khan); the comment on each
 * declaration names the reference interface it replaces.  The argument order follows the
 * reference functors (gpu_featurizer/functor_op.h:8-69): inputs, then outputs, then the
 * host-side `acs` array, then the stream.
 *
 * Conventions (all entry points):
 *  - every pointer is a DEVICE pointer unless the name ends in `_host`;
 *  - outputs are caller-allocated and, for every atom that a molecule range covers, fully
 *    written by the call: no pre-zeroing is needed (the reference zero-fills inside its
 *    functors, gpu_featurizer/functor_op_cpu.cpp:31-34).  Entries of atoms that belong to no
 *    molecule range are left as they were (feature rows) or unspecified (gradients): zero the
 *    arrays first if the molecule table does not cover the whole batch;
 *  - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = default stream)
 *    and the call returns without synchronising;
 *  - the return value is 0 (ANI_OK) or a negative ANI_ERR_* code; nothing calls exit()
 *    (the reference does, gpu_featurizer/functor_op_gpu.cu:12-20);
 *  - problems that only the device can see (an element id outside 0..3, a molecule range or
 *    scatter index outside the batch) are recorded in a per-device status word that
 *    ani_device_status() reads back; the offending atom/molecule is skipped or clamped,
 *    never dereferenced out of bounds;
 *  - n_atoms == 0 or n_mols == 0 is valid and does nothing (the reference trainer feeds
 *    empty batches on purpose, khan/training/trainer_multi_tower.py:796-817);
 *  - calls are re-entrant; concurrent calls on different streams/devices are independent.
 *
 * Element ids are the compacted ones of the reference: H 0, C 1, N 2, O 3.  The feature
 * row of an atom has ani_feature_size() = 384 entries: 64 radial then 320 angular
 * (gpu_featurizer/parameters.h:61-114).
 */
#ifndef ANI_B200_H_
#define ANI_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ANI_OK 0
#define ANI_ERR_NULL_POINTER (-1)   /* a required pointer argument is NULL              */
#define ANI_ERR_BAD_SIZE (-2)       /* negative count, or acs_host inconsistent          */
#define ANI_ERR_CUDA (-3)           /* a CUDA runtime call failed; see ani_last_cuda_error */
#define ANI_ERR_BAD_ELEMENT (-4)    /* device saw an element id outside 0..3 (status word) */
#define ANI_ERR_BAD_INDEX (-6)      /* device saw an offset/count/scatter index out of range */
#define ANI_ERR_TOO_MANY_ATOMS (-7) /* size beyond what an entry point supports          */
#define ANI_ERR_TIMEOUT (-8)        /* a bounded device-side wait ran out (status word)    */
#define ANI_ERR_MISALIGNED (-9)     /* a pointer that must be 16-byte aligned is not       */
#define ANI_ERR_CAPTURE (-10)       /* first-use set-up attempted while the stream is being captured */

/* Number of features per atom (384).  Replaces the `feature_size` attr of the Featurize op
 * (gpu_featurizer/ani_op.cpp:104). */
int ani_feature_size(void);

/* Text for a status code returned by any entry point. */
const char* ani_status_string(int status);

/* cudaGetErrorString of the last CUDA failure seen by this library on the calling thread. */
const char* ani_last_cuda_error(void);

/* Synchronises `stream`, then returns and clears the current device's status word:
 * ANI_OK or the first ANI_ERR_BAD_ELEMENT / ANI_ERR_BAD_INDEX seen by
 * a kernel since the last call.  No counterpart in the reference, which does not validate
 * its inputs (an element id outside 0..3 indexes out of bounds there,
 * gpu_featurizer/ani_sort.cpp:98-99). */
int ani_device_status(void* stream);

/*
 * AniSort -- replaces the CPU-only op of gpu_featurizer/ani_sort.cpp:71-115
 * (REGISTER_OP at :27-37).  Stable sort of the whole batch by element id:
 *   scatter_idxs[i] = rank of atom i among the atoms of its element, in batch order;
 *   gather_idxs[i]  = position of atom i in the element-sorted concatenation;
 *   atom_counts[4]  = atoms per element (device memory, 4 ints).
 * The input is read on the device (the reference reads it on the host).
 *
 * Up to 65,536 atoms the call is one launch and uses no memory beyond its arguments.  Larger
 * batches take three launches and a scratch buffer of (n_atoms / 1024 + 2) x 16 bytes that the
 * library allocates and keeps, one per (device, stream):
 *  - calls on different streams never share scratch, so they may overlap; calls on one stream
 *    run in stream order and share theirs;
 *  - the first large call on a stream (or the first one with more atoms than any before it)
 *    calls cudaMalloc: make it outside any stream capture -- inside one it is refused with
 *    ANI_ERR_CAPTURE and nothing is launched;
 *  - a buffer that is outgrown is replaced but not freed (a captured graph may still hold its
 *    address); all of them are released when the process ends.
 * ani_sort_noalloc below never allocates.
 */
int ani_sort(const int* atomic_numbers, int n_atoms, int* scatter_idxs, int* gather_idxs,
             int* atom_counts, void* stream);

/*
 * AniSort for callers that must not allocate.  It has no counterpart in the reference.
 *
 * ani_sort above may call cudaMalloc the first time a batch is too large for its
 * single-launch path (it caches a scratch buffer per device).  Some hosts cannot live with
 * that: a plugin whose execute call is forbidden to allocate, a process that has already
 * handed all device memory to a framework's pool, a latency-critical loop that cannot take
 * the device-wide synchronisation an allocation implies.  This variant computes exactly the
 * same three outputs with the same kernels, but its scratch (the per-tile element counts) is
 * a fixed array inside the library's own device data, so the call never allocates or frees
 * anything, on the device or through any library.
 *
 *  - Limit: n_atoms <= ani_sort_noalloc_max_atoms() (4,194,304); a larger batch is rejected
 *    with ANI_ERR_TOO_MANY_ATOMS before anything is launched.  The array costs 64 KiB of
 *    device memory on every GPU that loads the library, for the life of the process.
 *  - The first call on each device looks up the array's device address (with that device
 *    current) and remembers it; make that first call before any stream capture (a first call
 *    whose stream is being captured is refused with ANI_ERR_CAPTURE).
 *  - All calls on one device share the one array, and it keeps the previous call's contents.
 *    Every entry a call reads it has written first, so nothing needs clearing, but two calls
 *    that overlap on the GPU (different streams, or different host threads) race on it:
 *    keep calls on one device in one stream order.
 * Inputs and outputs are still the caller's buffers, as for ani_sort.
 */
int ani_sort_noalloc(const int* atomic_numbers, int n_atoms, int* scatter_idxs, int* gather_idxs,
                     int* atom_counts, void* stream);
int ani_sort_noalloc_max_atoms(void);

/*
 * Featurize -- replaces AniFunctor<Device, T> (gpu_featurizer/functor_op.h:8-25; CPU body
 * functor_op_cpu.cpp:13-43 -> featurize_cpu, kernel_cpu.cpp:406-537; GPU body
 * functor_op_gpu.cu:57-92 -> featurize, kernel.cu:72-268) and the op shell
 * AniCombined::Compute (gpu_featurizer/ani_op.cpp:29-92).
 *   xs, ys, zs [n_atoms], atomic_numbers [n_atoms], mol_offsets [n_mols],
 *   mol_atom_counts [n_mols], scatter_idxs [n_atoms] (from ani_sort),
 *   out_h/c/n/o: acs_host[t] * 384 values each, row-major rows of 384,
 *   acs_host: HOST array of 4 atom counts (HostMemory input of the op, ani_op.cpp:116).
 * An output whose acs_host[t] is 0 may be NULL.
 */
int ani_featurize_f32(const float* xs, const float* ys, const float* zs,
                      const int* atomic_numbers, const int* mol_offsets,
                      const int* mol_atom_counts, int n_mols, const int* scatter_idxs,
                      float* out_h, float* out_c, float* out_n, float* out_o,
                      const int* acs_host, void* stream);
int ani_featurize_f64(const double* xs, const double* ys, const double* zs,
                      const int* atomic_numbers, const int* mol_offsets,
                      const int* mol_atom_counts, int n_mols, const int* scatter_idxs,
                      double* out_h, double* out_c, double* out_n, double* out_o,
                      const int* acs_host, void* stream);

/*
 * FeaturizeGrad -- replaces AniGrad<Device, T> (gpu_featurizer/functor_op.h:27-47; CPU body
 * functor_op_cpu.cpp:48-83 -> featurize_grad_cpu, kernel_cpu.cpp:217-366) and
 * AniCombinedGrad::Compute (gpu_featurizer/ani_op.cpp:129-196).  The reference has no GPU
 * kernel for this op (ani_op.cpp:339-340).  Vector-Jacobian product: given dL/dfeatures in
 * the four per-element buffers, writes dL/dx, dL/dy, dL/dz [n_atoms].
 * Batches of small molecules (mean size <= 24 atoms) with 16-byte aligned grad_* buffers run one
 * CTA per molecule, every output written once and bit-reproducible from run to run; other
 * batches are accumulated with floating-point atomics (last bits may differ between runs).
 */
int ani_featurize_grad_f32(const float* xs, const float* ys, const float* zs,
                           const int* atomic_numbers, const int* mol_offsets,
                           const int* mol_atom_counts, int n_mols, const int* scatter_idxs,
                           const float* grad_h, const float* grad_c, const float* grad_n,
                           const float* grad_o, float* x_grads, float* y_grads, float* z_grads,
                           const int* acs_host, void* stream);
int ani_featurize_grad_f64(const double* xs, const double* ys, const double* zs,
                           const int* atomic_numbers, const int* mol_offsets,
                           const int* mol_atom_counts, int n_mols, const int* scatter_idxs,
                           const double* grad_h, const double* grad_c, const double* grad_n,
                           const double* grad_o, double* x_grads, double* y_grads,
                           double* z_grads, const int* acs_host, void* stream);

/*
 * FeaturizeGradInverse -- replaces AniGradInverse<Device, T> (gpu_featurizer/functor_op.h:49-69;
 * CPU body functor_op_cpu.cpp:88-121 -> featurize_grad_inverse, kernel_cpu.cpp:37-179) and
 * AniCombinedGradInverse (gpu_featurizer/ani_op.cpp:224-330), the op TensorFlow calls for the
 * second derivative through FeaturizeGrad (khan/training/trainer_multi_tower.py:64-91).
 * Jacobian-vector product: x_grads/y_grads/z_grads [n_atoms] is a displacement of every atom;
 * the outputs (same layout as Featurize) receive the directional derivative of every feature.
 * It is the exact transpose of ani_featurize_grad.  The reference kernel indexes the input
 * vector by the element id of the central atom (kernel_cpu.cpp:111-169), which makes its output
 * vanish up to rounding; this entry point computes the product that was meant.
 * Limit: at most 64 atoms within 4.6 A of any atom (else ANI_ERR_TOO_MANY_ATOMS in the status
 * word and a zero row).
 */
int ani_featurize_grad_inverse_f32(const float* xs, const float* ys, const float* zs,
                                   const int* atomic_numbers, const int* mol_offsets,
                                   const int* mol_atom_counts, int n_mols, const int* scatter_idxs,
                                   const float* x_grads, const float* y_grads, const float* z_grads,
                                   float* out_h, float* out_c, float* out_n, float* out_o,
                                   const int* acs_host, void* stream);
int ani_featurize_grad_inverse_f64(const double* xs, const double* ys, const double* zs,
                                   const int* atomic_numbers, const int* mol_offsets,
                                   const int* mol_atom_counts, int n_mols, const int* scatter_idxs,
                                   const double* x_grads, const double* y_grads,
                                   const double* z_grads, double* out_h, double* out_c,
                                   double* out_n, double* out_o, const int* acs_host, void* stream);

/*
 * Atomic networks, forward -- replaces the four AtomNN stacks that MoleculeNN builds
 * (khan/model/nn.py:39-67, 165-172) for the architecture 384-128-128-64-1 used by the
 * reference drivers (gdb8.py:91): for every element t,
 *   energy[t] = act(act(act(F_t W1 + b1) W2 + b2) W3 + b3) w4 + b4,   F_t = features[t] [acs[t]][384].
 * One launch covers all four elements; the matrix products run on the tensor cores in tf32.
 * Weights are passed as the reference stores them, [in][out] with `out` contiguous
 * (khan/model/nn.py:42-47).  Every matrix pointer (features, weights, act*, dact*) must be
 * 16-byte aligned (ANI_ERR_MISALIGNED otherwise).  `activation`: 0 celu(0.1),
 * 1 gaussian exp(-x^2), 2 normal exp(-x^2/2), 3 softplus - ln 2 (khan/model/activations.py:62-74).
 * `split_precision` != 0 splits every operand into two tf32 terms (three MMAs per product),
 * which brings the products to float32 accuracy; 0 uses plain tf32.
 * act1/act2/act3 receive the hidden activations ([acs[t]][128], [128], [64]) and
 * dact1/dact2/dact3 the derivatives of the activation function at the same places, when non-NULL
 * (the backward pass needs them).  Pointers of an element with acs_host[t] == 0 may be NULL.
 */
typedef struct ani_mlp_args {
    const float* features[4];
    const float* w1[4];   /* [384][128] */
    const float* b1[4];   /* [128] */
    const float* w2[4];   /* [128][128] */
    const float* b2[4];   /* [128] */
    const float* w3[4];   /* [128][64] */
    const float* b3[4];   /* [64] */
    const float* w4[4];   /* [64] */
    const float* b4[4];   /* [1] */
    float* energy[4];     /* [acs[t]] */
    float* act1[4];
    float* act2[4];
    float* act3[4];
    float* dact1[4];      /* optional: d act / d x at the same places (the backward pass needs them) */
    float* dact2[4];
    float* dact3[4];
    const void* packed[4];  /* optional: the same weights packed by ani_mlp_pack_weights_f32 */
} ani_mlp_args;

int ani_mlp_forward_f32(const ani_mlp_args* args_host, const int* acs_host, int activation,
                        int split_precision, void* stream);

/*
 * Optional pre-packing of the weights, no counterpart in the reference.  Writes, per element,
 * ani_mlp_packed_bytes() bytes (1.19 MiB) that hold W1, W2, W3 cut into the 32-column chunks of
 * both products that read them (forward: W^T; backward: W), split into tf32 high and low parts and
 * laid out as the tensor cores read them.  A forward / backward call that is given `packed`
 * fetches each chunk with one bulk asynchronous copy (TMA) instead of staging it with all threads;
 * results are identical.  The packed copy must be refreshed after every change of the weights;
 * elements whose packed[t] is NULL are skipped.  16-byte alignment required.
 */
typedef struct ani_mlp_pack_args {
    const float* w1[4];   /* [384][128] */
    const float* w2[4];   /* [128][128] */
    const float* w3[4];   /* [128][64] */
    void* packed[4];      /* ani_mlp_packed_bytes() each */
} ani_mlp_pack_args;

size_t ani_mlp_packed_bytes(void);
int ani_mlp_pack_weights_f32(const ani_mlp_pack_args* args_host, void* stream);

/*
 * Backward pass of the same four networks along the activations (float32), one launch:
 *   dz3 = (grad_energy w4^T) * dact3,  dz2 = (dz3 W3^T) * dact2,  dz1 = (dz2 W2^T) * dact1,
 *   grad_features = dz1 W1^T   (optional; this is the upstream of ani_featurize_grad).
 * It takes the place of the part of tf.gradients through MoleculeNN that reaches the features
 * (khan/model/nn.py:39-67,165-172 under khan/training/trainer_multi_tower.py:350-419).  The weight
 * gradients follow from the outputs as plain products over the atoms of an element,
 * dW_l = A_{l-1}^T dz_l and db_l = column sums of dz_l, and are left to the caller.
 * Weights are passed in the reference's layout, [in][out] with `out` contiguous; dact1..3 are the
 * arrays that ani_mlp_forward_f32 filled.  `split_precision` as in the forward call.  Every
 * matrix pointer must be 16-byte aligned (ANI_ERR_MISALIGNED otherwise).
 */
typedef struct ani_mlp_backward_args {
    const float* grad_energy[4];  /* [acs[t]] dL/dE per atom, element-sorted order */
    const float* w1[4];           /* [384][128] */
    const float* w2[4];           /* [128][128] */
    const float* w3[4];           /* [128][64] */
    const float* w4[4];           /* [64] */
    const float* dact1[4];        /* [acs[t]][128] */
    const float* dact2[4];        /* [acs[t]][128] */
    const float* dact3[4];        /* [acs[t]][64] */
    float* dz1[4];                /* [acs[t]][128] */
    float* dz2[4];                /* [acs[t]][128] */
    float* dz3[4];                /* [acs[t]][64] */
    float* grad_features[4];      /* [acs[t]][384], may be NULL */
    const void* packed[4];        /* optional: the same weights packed by ani_mlp_pack_weights_f32 */
} ani_mlp_backward_args;

int ani_mlp_backward_f32(const ani_mlp_backward_args* args_host, const int* acs_host,
                         int split_precision, void* stream);

/*
 * Weight and bias gradients of the same four networks, one launch, ADDED to the outputs (zero
 * them first, or pass gradient buffers that are being accumulated):
 *   dw1 += F^T dz1 [384][128],  dw2 += A1^T dz2 [128][128],  dw3 += A2^T dz3 [128][64],
 *   db1 += column sums of dz1,  db2 += ... dz2,  db3 += ... dz3,
 *   dw4 += A3^T g [64],  db4 += sum g   (g = grad_energy),
 * in the reference's weight layout ([in][out]); dw1, dw2, dw3 and every input matrix must be
 * 16-byte aligned (ANI_ERR_MISALIGNED otherwise).  features / act1..3 are the forward call's
 * input and saved activations, dz1..3 the outputs of ani_mlp_backward_f32.  Replaces the weight part of optimizer.compute_gradients through AtomNN
 * (khan/model/nn.py:39-67; khan/training/trainer_multi_tower.py:396-397).
 */
typedef struct ani_mlp_weight_grad_args {
    const float* features[4];  /* [acs[t]][384] */
    const float* act1[4];      /* [acs[t]][128] */
    const float* act2[4];      /* [acs[t]][128] */
    const float* dz1[4];       /* [acs[t]][128] */
    const float* dz2[4];       /* [acs[t]][128] */
    const float* dz3[4];       /* [acs[t]][64] */
    float* dw1[4];             /* [384][128] */
    float* dw2[4];             /* [128][128] */
    float* dw3[4];             /* [128][64] */
    float* db1[4];             /* [128] */
    float* db2[4];             /* [128] */
    float* db3[4];             /* [64] */
    const float* act3[4];      /* [acs[t]][64] */
    const float* grad_energy[4];   /* [acs[t]] */
    float* dw4[4];             /* [64] */
    float* db4[4];             /* [1] */
} ani_mlp_weight_grad_args;

int ani_mlp_weight_grad_f32(const ani_mlp_weight_grad_args* args_host, const int* acs_host,
                            int split_precision, void* stream);

/*
 * Molecule energies and the squared-error loss -- replaces tf.gather + tf.segment_sum + the
 * squared difference of khan/model/nn.py:171-172 and khan/training/trainer_multi_tower.py:350,390-392.
 *   mol_energy[m] = sum over the atoms i of molecule m of atom_energy_sorted[gather_idxs[i]]
 * (atom_energy_sorted is in the element-sorted order in which the networks produce it,
 * gather_idxs as returned by ani_sort).  With `labels` (one target per molecule):
 *   l2s[m] = (mol_energy[m] - labels[m])^2                                   (if l2s != NULL)
 *   grad_atom_energy_sorted[gather_idxs[i]] = grad_scale * 2 (mol_energy[m] - labels[m])
 * i.e. with grad_scale = 1 / n_mols the derivative of the mean squared error with respect to
 * every atomic energy, in the order ani_mlp_backward_f32 reads it (if != NULL; entries of atoms
 * outside every molecule are left untouched).  One warp per molecule, no atomics.
 */
int ani_molecule_energy_f32(const float* atom_energy_sorted, const int* gather_idxs, const int* mol_offsets,
                            const int* mol_atom_counts, int n_mols, int n_atoms, const float* labels,
                            float grad_scale, float* mol_energy, float* l2s, float* grad_atom_energy_sorted,
                            void* stream);

/*
 * One optimiser step over a flat float32 weight buffer, two launches: global-norm clipping,
 * Adam with Nesterov momentum, and the exponential moving average of the weights.  It takes the
 * place of tf.clip_by_global_norm + NadamOptimizer.apply_gradients +
 * ExponentialMovingAverage.apply of khan/training/trainer_multi_tower.py:261-266,421-427:
 *   g <- g * c / max(||g||, c);  m <- b1 m + (1-b1) g;  v <- b2 v + (1-b2) g^2;
 *   w <- w - lr sqrt(1-b2^t)/(1-b1^t) (b1 m + (1-b1) g) / (sqrt(v) + eps);
 *   ema <- ema - (1-d)(ema - w),  d = min(ema_decay, (1+t)/(10+t)),   t = steps so far + 1.
 * `hyper` is DEVICE memory, six floats {lr, beta1, beta2, eps, clip_norm, ema_decay}
 * (clip_norm <= 0 disables clipping); `state` is 32 bytes of DEVICE memory that the caller
 * zero-fills once (step counter and scratch; the step counter is its first int).  `ema` may be
 * NULL.  Nothing is read on the host, so the call can be captured into a CUDA graph.
 */
int ani_nadam_step_f32(float* params, const float* grads, float* m, float* v, float* ema,
                       long long n, const float* hyper, void* state, void* stream);

/*
 * Max-norm constraint on weight rows, one launch: row r is params[row_offsets[r] ..
 * row_offsets[r] + row_lengths[r]); a row whose Euclidean norm exceeds max_norm is scaled to
 * norm max_norm.  Replaces the list of tf.assign(w, tf.clip_by_norm(w, 3.0, axes=1)) ops that
 * the reference runs before every training batch (khan/training/trainer_multi_tower.py:432-436,
 * `before_hooks=self.max_norm_ops` at :851).  row_offsets / row_lengths are device arrays.
 */
int ani_clip_rows_f32(float* params, const int* row_offsets, const int* row_lengths, int n_rows, float max_norm,
                      void* stream);

/*
 * The gradient of the reference's training losses from the gradient of the mean squared error, one launch:
 * grads[0 .. n) *= 1 / (2 rmse)  (kind 1: the rmse loss)  or  exp(rmse) / (2 rmse)  (kind 2: exp(rmse), the
 * loss khan minimises, khan/training/trainer_multi_tower.py:390-396), rmse = sqrt(mean(l2s[0 .. n_mols))),
 * formed on the device; rmse_out (one float, device; may be NULL) receives it.
 */
int ani_scale_by_loss_f32(float* grads, long long n, const float* l2s, int n_mols, int kind, float* rmse_out,
                          void* stream);

/*
 * AniCharge -- replaces the op of gpu_featurizer/ani_charges.cpp:45-56,58-113 (CPU, float and
 * double) and gpu_featurizer/ani_charges_gpu.cu:60-128 (GPU, float only).  Damped Coulomb
 * energy of every molecule,
 *   charge_energies[m] = k_e * sum_{i<j in m} q_i q_j (1 - f_C(r_ij, R_Rc)) / r_ij ,
 * k_e = 0.529176917 (gpu_featurizer/parameters.h:10).  `qs` holds one partial charge per atom.
 * n_atoms is the length of xs/ys/zs/qs and is used only to validate the molecule table
 * (the reference takes it from the tensor shape and does not check).
 */
int ani_charge_f32(const float* xs, const float* ys, const float* zs, const float* qs,
                   const int* mol_offsets, const int* mol_atom_counts, int n_mols, int n_atoms,
                   float* charge_energies, void* stream);
int ani_charge_f64(const double* xs, const double* ys, const double* zs, const double* qs,
                   const int* mol_offsets, const int* mol_atom_counts, int n_mols, int n_atoms,
                   double* charge_energies, void* stream);

/*
 * AniChargeGrad -- replaces gpu_featurizer/ani_charges.cpp:123-135,138-214 and
 * gpu_featurizer/ani_charges_gpu.cu:197-260: q_grads[i] = grads[m(i)] * dE_m/dq_i, the gradient
 * that the reference registers for AniCharge (khan/training/trainer_multi_tower.py:94-120).
 * q_grads (n_atoms values) is zero-filled by the call; atoms outside every molecule keep 0.
 * Molecule ranges must not overlap (the reference would add the contributions up).
 */
int ani_charge_grad_f32(const float* xs, const float* ys, const float* zs, const float* qs,
                        const int* mol_offsets, const int* mol_atom_counts, int n_mols, int n_atoms,
                        const float* grads, float* q_grads, void* stream);
int ani_charge_grad_f64(const double* xs, const double* ys, const double* zs, const double* qs,
                        const int* mol_offsets, const int* mol_atom_counts, int n_mols, int n_atoms,
                        const double* grads, double* q_grads, void* stream);

/*
 * Host-side batch assembly (no CUDA call, usable without a GPU): writes the batch made of the
 * molecules picks[0..n_picks) of a packed dataset, in that order, into one host arena -- what
 * RawDataset.iterate of the reference builds with a Python loop over molecules and
 * np.concatenate (khan/data/dataset.py:144-183) and what the reference's feed then copies
 * (khan/training/trainer_multi_tower.py:749-828).
 *
 * Source (the packed dataset): mol_ptr[n_mols_total + 1] is the CSR of atom ranges; src_xyz is
 * [3][src_stride] in float (src_is_f64 = 0) or double; src_types[...] element ids; src_ys
 * (optional) one label per molecule and src_grads (optional) [3][src_stride], both in the
 * DESTINATION precision.  noise (optional): [atoms of the batch][3] doubles added to the
 * coordinates before the cast, the sum formed in double (the coordinate fuzz of
 * RawDataset.iterate, drawn by the caller so that the random stream stays numpy's).
 * Destination: dst_xyz / dst_grads [3][dst_stride] and dst_ys in float (dst_is_f64 = 0) or
 * double, dst_types[cap_atoms], dst_mol_ids[cap_atoms] (index of the molecule within the batch),
 * dst_mol_offsets / dst_mol_counts[cap_mols].  n_atoms_out receives the atoms of the batch and
 * acs_out[4] the atoms per element.  ANI_ERR_BAD_SIZE if the batch does not fit cap_atoms /
 * cap_mols (nothing is written then), ANI_ERR_BAD_INDEX for a pick outside the dataset.
 */
typedef struct ani_host_pack_args {
    const long long* picks;
    int n_picks;
    long long n_mols_total;
    const long long* mol_ptr;
    const void* src_xyz;
    long long src_stride;
    int src_is_f64;
    const int* src_types;
    const void* src_ys;
    const void* src_grads;
    const double* noise;
    void* dst_xyz;
    void* dst_grads;
    void* dst_ys;
    long long dst_stride;
    int dst_is_f64;
    int* dst_types;
    long long* dst_mol_ids;
    int* dst_mol_offsets;
    int* dst_mol_counts;
    int cap_atoms;
    int cap_mols;
    int* n_atoms_out;
    int* acs_out;
    const int* src_mol_acs;   /* optional [n_mols_total][4]: atoms per element of every molecule of the dataset;
                                 when given, the per-batch element counts are sums of these rows */
} ani_host_pack_args;
int ani_host_pack_batch(const ani_host_pack_args* args);

/*
 * One pass over a staged batch as ONE call: any run of the steps
 *   pack weights -> ani_sort -> featurize -> networks forward -> molecule energies (+ MSE gradient)
 *   -> networks backward -> zero + weight gradients -> featurize_grad
 * chosen by `phases`, each step the entry point of that name above, enqueued in this order on
 * `stream`.  It has no counterpart in the reference, where TensorFlow's executor walks the graph
 * of trainer_multi_tower.py:290-427; it exists because the host-side cost of six to eight separate
 * calls, each with its own argument block of per-element pointers, is what bounds predict /
 * coordinate_gradients / feed_dataset from Python.  All row buffers hold the atoms in the
 * element-sorted order of ani_sort (H rows, then C, N, O); the per-element pointers of the single
 * calls are these bases plus the element's row offset, computed here from acs_host.
 */
#define ANI_PASS_PACK 1          /* ani_mlp_pack_weights_f32 (needs `packed`) */
#define ANI_PASS_FEATURIZE 2     /* ani_sort + ani_featurize_f32 */
#define ANI_PASS_FORWARD 4       /* ani_mlp_forward_f32 */
#define ANI_PASS_ENERGY 8        /* ani_molecule_energy_f32 (with labels: l2s and grad_energy_sorted are written) */
#define ANI_PASS_BACKWARD 16     /* ani_mlp_backward_f32 (feature_grads == NULL skips the products towards the features) */
#define ANI_PASS_WEIGHT_GRAD 32  /* clear zero_ptr[0 .. zero_bytes), then ani_mlp_weight_grad_f32 */
#define ANI_PASS_COORD_GRAD 64   /* ani_featurize_grad_f32 with feature_grads as its upstream */
typedef struct ani_pass_args {
    int phases;
    int n_atoms, n_mols;
    const int* acs_host;             /* HOST [4] */
    int activation, split_precision;
    const float *xs, *ys, *zs;       /* [n_atoms] */
    const int *atomic_numbers, *mol_offsets, *mol_atom_counts;
    int *scatter_idxs, *gather_idxs, *atom_counts;
    float* features;                 /* [n_atoms][384] */
    float* feature_grads;            /* [n_atoms][384] or NULL */
    float *x_grads, *y_grads, *z_grads;
    float* energy_sorted;            /* [n_atoms] */
    float* grad_energy_sorted;       /* [n_atoms]: read by the backward steps, written by the energy step when labels != NULL */
    float *act1, *act2, *act3;       /* [n_atoms][128], [128], [64] */
    float *dact1, *dact2, *dact3;
    float *dz1, *dz2, *dz3;
    const float* labels;             /* [n_mols] or NULL */
    float grad_scale;
    float* mol_energy;               /* [n_mols] */
    float* l2s;                      /* [n_mols] or NULL */
    const float *w1[4], *b1[4], *w2[4], *b2[4], *w3[4], *b3[4], *w4[4], *b4[4];
    float *dw1[4], *db1[4], *dw2[4], *db2[4], *dw3[4], *db3[4], *dw4[4], *db4[4];
    void* packed[4];                 /* pre-packed weights per element, or NULL */
    void* zero_ptr;                  /* cleared before the weight gradients are added (NULL: nothing) */
    size_t zero_bytes;
} ani_pass_args;
int ani_network_pass_f32(const ani_pass_args* args, void* stream);

/*
 * The submitter thread of the batch feeder in native code (the reference: a Python thread that
 * pushes feed_dicts into a TensorFlow FIFOQueue, khan/training/trainer_multi_tower.py:749-828,
 * over batches assembled by khan/data/dataset.py:144-183).  A feeder owns a ring of slots; a slot
 * is one pinned HOST arena laid out by the caller (the dst_* pointers of `pack` point into it),
 * its DEVICE twin of the same size, and the source pointers of the packed data set (src_*,
 * mol_ptr, n_mols_total, cap_* of `pack`; picks, noise and the *_out fields are set by the feeder).
 * One pass:
 *   ani_feeder_begin(f, order, n, batch_size)   batch b = molecules order[b*batch_size ...) of the
 *                                               data set; starts the thread, which packs batch
 *                                               after batch into free slots (ani_host_pack_batch)
 *                                               and enqueues ONE host-to-device copy of the arena
 *                                               per batch on the feeder's own copy stream
 *   ani_feeder_next(f, &b)     blocks until the next batch is packed and its copy enqueued;
 *                              returns 1 (a batch), 0 (pass over) or a negative ANI_ERR_* of the thread
 *   ani_feeder_wait(f, slot, stream)      `stream` waits for that batch's copy
 *   ani_feeder_release(f, slot, stream)   the slot may be refilled; the next copy into its device
 *                                         arena is ordered behind the work enqueued on `stream` so far
 *   ani_feeder_end(f)          stops the thread (idempotent; begin() calls it first)
 * device < 0: host only -- no CUDA call is made, the consumer reads the host arenas (stream unused).
 * A slot's arenas must outlive the feeder; ani_feeder_destroy waits for the copies still in flight.
 * Calls on one feeder come from one consumer thread.
 */
typedef struct ani_feeder_slot {
    ani_host_pack_args pack;
    void* host_arena;   /* pinned when device >= 0 */
    void* dev_arena;    /* NULL when device < 0 */
    size_t nbytes;      /* bytes copied per batch (the whole arena) */
} ani_feeder_slot;
typedef struct ani_feeder_batch {
    int slot;
    long long batch_index;
    int n_atoms, n_mols;
    int acs[4];         /* atoms per element: what ani_sort returns as atom_counts */
} ani_feeder_batch;
typedef struct ani_feeder ani_feeder;
int ani_feeder_create(int device, const ani_feeder_slot* slots, int n_slots, ani_feeder** out);
int ani_feeder_begin(ani_feeder* f, const long long* order, long long n_order, int batch_size);
int ani_feeder_next(ani_feeder* f, ani_feeder_batch* out);
int ani_feeder_wait(ani_feeder* f, int slot, void* stream);
int ani_feeder_release(ani_feeder* f, int slot, void* stream);
int ani_feeder_end(ani_feeder* f);
int ani_feeder_destroy(ani_feeder* f);

/*
 * Mean of a float buffer over the GPUs of one node through peer memory, one kernel launch per rank
 * and call: the average of the weight gradients over the towers (the reference: per-variable concat
 * + reduce_mean on the CPU, khan/training/trainer_multi_tower.py:137-179).  One process per GPU;
 * every rank creates a handle of the same capacity, the ranks exchange the 64-byte handles of their
 * blocks (any host transport) and connect; from then on every rank calls ani_peer_mean_f32 the same
 * number of times with buffers of the same length, and each call leaves the SAME mean, bit for bit,
 * on every rank.  Launch only: it can be captured in a CUDA graph (the step number lives in device
 * memory).  Calls on one handle must be ordered (one stream).  The wait for the other ranks is
 * bounded (a fraction of a second by default): when it runs out, the call still ends, the result
 * of that step is unspecified and ani_device_status reports ANI_ERR_TIMEOUT.
 *   n: floats in the buffer, a multiple of 4, at most the capacity; buffer 16-byte aligned.
 *   ani_peer_connect_raw / ani_peer_block: for ranks that live in one process (the peer's block by
 *   address instead of by handle).  ani_peer_destroy synchronises the device first.
 */
typedef struct ani_peer ani_peer;
int ani_peer_create(int rank, int world, long long n_floats, ani_peer** out);
int ani_peer_handle(ani_peer* p, void* out64);
int ani_peer_connect(ani_peer* p, int rank_q, const void* handle64);
int ani_peer_connect_raw(ani_peer* p, int rank_q, void* block);
void* ani_peer_block(ani_peer* p);
int ani_peer_set_spin_limit(ani_peer* p, unsigned tries);
int ani_peer_set_two_halves(ani_peer* p, int on);   /* on: every rank forms the mean of its slice and the slices are
                                                       exchanged (default for more than four ranks); off: every rank
                                                       sums everything.  The same setting on every rank. */
int ani_peer_mean_f32(ani_peer* p, float* buffer, long long n, void* stream);
int ani_peer_destroy(ani_peer* p);

#ifdef __cplusplus
}
#endif
#endif /* ANI_B200_H_ */
