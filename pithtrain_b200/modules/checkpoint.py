"""placeholder replaced below"""


def save_training_checkpoint(cfg):
    raise NotImplementedError


def load_training_checkpoint(cfg):
    if cfg.training.save_location is None:
        return
    raise NotImplementedError
