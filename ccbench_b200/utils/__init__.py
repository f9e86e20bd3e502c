"""Host utilities: clock sampling, NUMA binding, environment description, persistent state."""
