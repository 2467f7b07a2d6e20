"""Process groups, explicit tensor/sequence-parallel collectives, symmetric memory and the
sharded-data-parallel (FSDP-style) runtime."""
