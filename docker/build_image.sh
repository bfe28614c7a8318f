#!/usr/bin/env bash
# Build the serving image from the repository root:  docker/build_image.sh [tag]
set -euo pipefail
cd "$(dirname "$0")/.."
TAG="${1:-vllm-metax-b200:$(python3 -c 'import re;print(re.search(r"__version__ = \"(.*)\"", open("vllm_metax_b200/version.py").read()).group(1))')}"
docker build -f docker/b200.Dockerfile -t "$TAG" .
echo "built $TAG"
