"""The ``art`` package name resolves to the same modules as ``art_b200``."""


def test_import_art_alias():
    import art
    import art_b200

    assert art.TrainableModel is art_b200.TrainableModel
    assert art.Trajectory is art_b200.Trajectory
    assert art.gather_trajectory_groups is art_b200.gather_trajectory_groups
    from art.local import LocalBackend
    from art_b200.local import LocalBackend as L2

    assert LocalBackend is L2
    import art.dev as dev
    import art.utils.benchmarking.types as bt
    import art_b200.utils.benchmarking.types as bt2

    assert bt is bt2 and hasattr(dev, "TrainConfig")
    from art.utils import iterate_dataset, retry  # noqa: F401
