"""Native sampling maskers."""
