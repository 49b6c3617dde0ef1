"""Host-side utilities: RNG / data sources, arena layout, CKP1 and CHRN file IO, CLI flags."""
