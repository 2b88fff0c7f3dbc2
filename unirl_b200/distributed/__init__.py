"""Distributed runtime: device pool, placement, handles/workers, tensor transport, weight sync."""
