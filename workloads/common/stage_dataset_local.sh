#!/bin/bash
# Copy a dataset directory to node-local storage once per node: rsync, then a .stage_complete
# sentinel holding the source path and byte count; a later call with the same source is a no-op.
set -euo pipefail
SRC="${1:?source dir}"; DST="${2:?destination dir}"
SENTINEL="${DST}/.stage_complete"
if [ -f "${SENTINEL}" ] && [ "$(head -n1 "${SENTINEL}")" = "${SRC}" ]; then
  echo "dataset already staged at ${DST}"; exit 0
fi
mkdir -p "${DST}"
if command -v rsync >/dev/null 2>&1; then rsync -a --delete "${SRC}/" "${DST}/"; else cp -a "${SRC}/." "${DST}/"; fi
bytes=$(du -sb "${DST}" | cut -f1)
printf '%s\n%s\n' "${SRC}" "${bytes}" > "${SENTINEL}"
echo "staged ${bytes} bytes to ${DST}"
