"""Model packages.  Each = config + bundle + conditions + stages + pipeline."""
