// cleanup_* of a GPU competitor hands P back with S's pattern (the reference's convention, e.g.
// src/competitors/gpu/gpu_convert.hpp:58-64).  The containers only offer copying setters for the index arrays
// (src/matrices/CSR.hpp:125-139, src/matrices/COO.hpp:149-163), 150 MB each on the largest configuration: the copies
// run on helper threads beside the device-to-host copy of the values instead of after it.
#pragma once
#include <thread>

namespace SDDMM {

// P takes S's index arrays on two helper threads while `download` (which fills P's values) runs on the caller's.
template <class Sparse, class Download>
void finish_into(Sparse &S, Sparse &P, Download &&download) {
    if (P.getValues().size() != S.getValues().size()) P.getValues().resize(S.getValues().size());
    std::thread cols([&] { P.setColPositions(S.getColPositions()); });
    std::thread rows([&] { P.setRowPositions(S.getRowPositions()); });
    download(P.getValues().data());
    cols.join();
    rows.join();
}

}  // namespace SDDMM
