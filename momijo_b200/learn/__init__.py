"""momijo.learn API family (nn, losses, optim, data, distributed, engine, callbacks, api, ...)."""
