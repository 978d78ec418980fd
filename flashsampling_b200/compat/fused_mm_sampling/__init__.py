"""Import shim: the reference's package name, backed by flashsampling_b200 (fused path only)."""
