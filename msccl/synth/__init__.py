"""Synthesis core: SMT path encoding, lower bounds, duality reduction, isomorphisms, search."""
