"""Framework utilities: low-precision parameter shadows, device timers, checkpoint IO, logging."""
