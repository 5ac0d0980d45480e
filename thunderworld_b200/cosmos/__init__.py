"""Plan loading, issued-work accounting, W1-support storage and the graph-capture contract of the
joint-inference runtime (reference package: thunderworld_fp4.cosmos)."""
