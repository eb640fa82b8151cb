"""Python boundary of the serving path: the same names and call shapes as
TileMega's python/tilemega/serving (plan, state, weights, engine)."""
