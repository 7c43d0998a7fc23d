"""Import stub: the reference's neon frontend imports h5py at module level for its callbacks;
nothing here writes HDF5 files."""
