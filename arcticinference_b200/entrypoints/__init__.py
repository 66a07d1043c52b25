"""Network entry points: the OpenAI-compatible server and the command line."""
