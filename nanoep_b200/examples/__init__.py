"""Runnable examples."""
