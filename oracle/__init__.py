"""CPU oracle of the SparseLinear hot path. Test infrastructure; never imported by the product."""
