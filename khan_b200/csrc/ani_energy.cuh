// Molecule energies from atomic energies, and the derivative of the mean-squared-error loss with
// respect to the atomic energies, in one kernel.
//
// The reference sums the atomic energies per molecule with tf.segment_sum
// (khan/training/trainer_multi_tower.py:350) after gathering them back from the element-sorted
// order (khan/model/nn.py:171-172), and forms (E_mol - y)^2 per molecule (:390-392).  Here one
// warp takes one molecule: its lanes gather the atomic energies of the molecule's atoms through
// gather_idxs, a shuffle reduction gives E_mol (no atomics: bit-reproducible), and, when labels
// are given, the warp writes the squared error and scatters dL/dE_atom = grad_scale * 2 (E_mol - y)
// back to the element-sorted positions, which is the input of the network backward pass.
#pragma once

#include "ani_common.cuh"

namespace ani {

template <int NW>
__global__ void __launch_bounds__(NW* kWarp)
    molecule_energy_kernel(const float* __restrict__ atom_energy_sorted, const int* __restrict__ gather,
                           const int* __restrict__ mol_offsets, const int* __restrict__ mol_counts,
                           int n_mols, int n_atoms, const float* __restrict__ labels, float grad_scale,
                           float* __restrict__ mol_energy, float* __restrict__ l2s,
                           float* __restrict__ grad_atom_energy_sorted)
{
    const int lane = lane_id();
    const int grid_warps = gridDim.x * NW;
    for (int m = blockIdx.x * NW + warp_id(); m < n_mols; m += grid_warps) {
        MolRange mol;
        float e = 0.0f;
        const bool ok = load_molecule(mol_offsets, mol_counts, m, n_atoms, &mol);
        if (ok) {
            for (int i = lane; i < mol.n; i += kWarp) {
                const int g = gather[mol.base + i];
                if (g >= 0 && g < n_atoms) e += atom_energy_sorted[g];
                else report(ANI_ERR_BAD_INDEX);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) e += __shfl_xor_sync(kFull, e, o);
        }
        if (lane == 0) mol_energy[m] = e;
        if (labels) {
            const float diff = e - labels[m];
            if (lane == 0 && l2s) l2s[m] = diff * diff;
            if (ok && grad_atom_energy_sorted) {
                const float g_mol = grad_scale * 2.0f * diff;
                for (int i = lane; i < mol.n; i += kWarp) {
                    const int g = gather[mol.base + i];
                    if (g >= 0 && g < n_atoms) grad_atom_energy_sorted[g] = g_mol;
                }
            }
        }
    }
}

}  // namespace ani
