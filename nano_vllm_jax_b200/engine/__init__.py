"""Host-side prefix reuse, batch layouts and GDN hybrid-state snapshots."""
