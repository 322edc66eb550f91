"""Training / evaluation loops."""
