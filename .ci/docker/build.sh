#!/usr/bin/env bash
# Usage: .ci/docker/build.sh [tag]   (run from the repository root)
set -euo pipefail
tag="${1:-torchtitan-b200:dev}"
docker build -f .ci/docker/Dockerfile -t "${tag}" .
echo "built ${tag}"
