"""vLLM serving glue: request router, per-node server controller and the client used by trainers."""
