"""Serving-engine integrations."""
