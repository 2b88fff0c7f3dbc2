"""Train side: sharded backend, train stack, adapter injection, EMA."""
