"""Scheduler, step function, engine handle, trace replay."""
