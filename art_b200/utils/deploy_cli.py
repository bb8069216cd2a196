"""``deploy-model`` command: pull a model's checkpoint(s) from the backup bucket and deploy one step as a serverless
LoRA (parity: the reference's ``scripts/deploy-model.py:19-108``; the pull / step selection order is the same: with
``--step latest`` every checkpoint is pulled first so that the newest step is known, otherwise only the one asked for).

    deploy-model --project my-project --model agent-001 --base-model Qwen/Qwen2.5-14B-Instruct --step latest
"""
from __future__ import annotations

import argparse
import asyncio
import os


def parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(description="Deploy a trained LoRA checkpoint to a hosted inference provider")
    ap.add_argument("--project", required=True)
    ap.add_argument("--model", required=True, help="name of the trained model")
    ap.add_argument("--base-model", required=True)
    ap.add_argument("--backup-bucket", default=None, help="S3 bucket with the checkpoints (default: $BACKUP_BUCKET)")
    ap.add_argument("--step", default="latest", help='checkpoint step, or "latest"')
    ap.add_argument("--art-path", default=".art")
    ap.add_argument("--provider", default="together")
    return ap.parse_args(argv)


async def deploy(args: argparse.Namespace, *, pull=None, deploy_fn=None):
    """``pull`` / ``deploy_fn`` default to the S3 and provider functions of this package (tests pass fakes)."""
    from .. import TrainableModel
    from .deploy_model import deploy_model
    from .get_model_step import get_model_step
    from .s3 import pull_model_from_s3

    pull = pull or pull_model_from_s3
    deploy_fn = deploy_fn or deploy_model
    bucket = args.backup_bucket or os.environ.get("BACKUP_BUCKET")
    if not bucket:
        raise SystemExit("no bucket: pass --backup-bucket or set BACKUP_BUCKET")
    model = TrainableModel(name=args.model, project=args.project, base_model=args.base_model)
    if args.step == "latest":
        print("Pulling all checkpoints to find the latest step ...")
        await pull(model_name=model.name, project=model.project, art_path=args.art_path, s3_bucket=bucket)
        step = get_model_step(model, args.art_path)
    else:
        step = int(args.step)
        print(f"Pulling the checkpoint of step {step} ...")
        await pull(model_name=model.name, project=model.project, art_path=args.art_path, s3_bucket=bucket, step=step)
    print(f"Deploying {args.model} (project {args.project}, step {step}) from s3://{bucket} ...")
    job = await deploy_fn(deploy_to=args.provider, model=model, step=step, verbose=True, pull_s3=False,
                          wait_for_completion=True, art_path=args.art_path)
    if str(getattr(job.status, "value", job.status)) == "Failed":
        raise RuntimeError(f"Deployment failed: {job.failure_reason}")
    print(f"Deployed as {job.model_name} (job {job.job_id})")
    return job


def main(argv: list[str] | None = None) -> None:
    asyncio.run(deploy(parse_args(argv)))


if __name__ == "__main__":
    main()
