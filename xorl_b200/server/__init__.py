"""Server mode: REST training service (forward_backward / optim_step futures), orchestrator,
worker runner, weight sync to an inference engine."""
