"""Controller-side trainers: generate → score → advantage → update → sync."""
