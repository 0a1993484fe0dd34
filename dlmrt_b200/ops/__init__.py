"""Host-side mirrors of the reference's `dlmrt/ops` modules that the row-parallel hot path lives inside."""
