// TEST INFRASTRUCTURE ONLY: C entry point around the reference's own CPU
// functor for IndexReplacer, compiled from the HGCalML checkout.
#include <cmath>
#include "index_replacer_kernel.cc"

extern "C" void ref_index_replacer(
        const int *to_be_replaced, const int *replacements, int *replaced,
        int n_to_be_replaced, int n_replacements) {
    tensorflow::functor::IndexReplacerOpFunctor<tensorflow::CPUDevice, int>()(
            tensorflow::CPUDevice(), to_be_replaced, replacements, replaced,
            n_to_be_replaced, n_replacements);
}
