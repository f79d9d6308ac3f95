// TEST INFRASTRUCTURE ONLY: C entry point around the reference's own CPU
// functor for BinnedAssignToCondensates, compiled from the HGCalML checkout.
// The functor can throw std::runtime_error (its progress guard); that is
// turned into a return code so nothing propagates through the C boundary.
#include <cmath>
#include "binned_assign_to_condensates_kernel.cc"

extern "C" int ref_binned_assign_to_condensates(
        int dimensions, int dimensions_binning,
        int *condensates_assigned_h,
        const float *ccoords_h, const float *dist_h, const float *beta_h,
        const int *no_condensation_mask_h,
        int *high_assigned_status_h,
        const int *original_indices_h, const int *row_splits_h,
        const float *ccoords, const float *dist, const int *no_condensation_mask,
        const int *indices_to_filtered,
        float *assignment_min_distance,
        int *assignment, int *association, int *n_condensates, int *alpha_indices,
        const int *bin_splits, const int *n_bins, const float *bin_widths,
        const int *row_splits, int num_rows, int assign_by_max_beta) {
    try {
        tensorflow::functor::BinnedCondensatesFinderOpFunctor<tensorflow::CPUDevice, int>()(
                tensorflow::CPUDevice(), dimensions, dimensions_binning,
                condensates_assigned_h, ccoords_h, dist_h, beta_h, no_condensation_mask_h,
                high_assigned_status_h, original_indices_h, row_splits_h,
                ccoords, dist, no_condensation_mask, indices_to_filtered,
                assignment_min_distance, assignment, association, n_condensates, alpha_indices,
                bin_splits, n_bins, bin_widths, row_splits, num_rows, assign_by_max_beta != 0);
    } catch (const std::exception &) {
        return -1;
    }
    return 0;
}
