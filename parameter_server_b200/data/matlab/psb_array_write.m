function psb_array_write(path, a, type)
% PSB_ARRAY_WRITE  Write an array as a raw little-endian file of the given element type (default: class of a).
% Counterpart of the reference's save_bin.m (src/data/matlab/save_bin.m).
  if nargin < 3, type = class(a); end
  fid = fopen(path, 'w', 'ieee-le');
  if fid < 0, error('psb:io', 'cannot create %s', path); end
  closer = onCleanup(@() fclose(fid));
  n = fwrite(fid, a(:), type);
  if n ~= numel(a), error('psb:io', 'short write to %s (%d of %d)', path, n, numel(a)); end
end
