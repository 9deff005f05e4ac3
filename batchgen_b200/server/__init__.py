"""OpenAI-style batch HTTP server, control plane (intake / scheduling pools, batch scheduler, worker manager,
watchdog) and the Python client."""
