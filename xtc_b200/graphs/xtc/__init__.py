"""Graph DSL (mirror of the reference's ``xtc.graphs.xtc``)."""
