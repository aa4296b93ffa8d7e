"""Host-side helpers: tile reordering, config files, timing, clocks."""
