function psb_write_text(path, y, X, varargin)
% PSB_WRITE_TEXT  Write labels y and sparse features X as text, one example per line (small data, for checks).
%   psb_write_text(path, y, X)                        LIBSVM: "label id:value id:value ..."  (ids 1-based as stored)
%   psb_write_text(path, y, X, 'group_id', g)         grouped: "label; g1 id[:value] ...; g2 ...;" with 0-based ids;
%                                                     g(c) is the group of column c and must be non-decreasing
%   psb_write_text(..., 'binary', true)               ids only
% Counterpart of the reference's saveas_pserver.m (src/data/matlab/saveas_pserver.m).
  p = inputParser;
  addParameter(p, 'group_id', []); addParameter(p, 'binary', false);
  parse(p, varargin{:}); o = p.Results;
  if ~isempty(o.group_id) && ~issorted(o.group_id), error('psb:arg', 'group_id must be sorted'); end
  fid = fopen(path, 'w');
  if fid < 0, error('psb:io', 'cannot create %s', path); end
  closer = onCleanup(@() fclose(fid));
  Xt = X';                                                        % one example per column: cheap to slice
  for r = 1:numel(y)
    [c, ~, v] = find(Xt(:, r));
    fprintf(fid, '%g', y(r));
    if isempty(o.group_id)
      for k = 1:numel(c)
        if o.binary, fprintf(fid, ' %d', c(k)); else, fprintf(fid, ' %d:%g', c(k), v(k)); end
      end
      fprintf(fid, '\n');
    else
      last = NaN;
      for k = 1:numel(c)
        g = o.group_id(c(k));
        if ~isequal(g, last), fprintf(fid, '; %d', g); last = g; end
        if o.binary, fprintf(fid, ' %d', c(k) - 1); else, fprintf(fid, ' %d:%g', c(k) - 1, v(k)); end
      end
      fprintf(fid, ';\n');
    end
  end
end
